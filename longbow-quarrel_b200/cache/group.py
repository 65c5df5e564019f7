"""What a group of cache entries with one need looks like to the cache.

The cache knows slots and lengths; each group knows its own storage.  A mixer's need
(`parts.base.CacheNeed`) makes its group, so a mixer with storage of another shape
than the two kinds that live here (paged keys and values, fixed-size state) brings a
class derived from `CacheGroup` with it and no file of the cache changes.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class CacheSizing:
    """How large the cache is: `n_pages` pages of `page_size` tokens for all live sequences together,
    at most `pages_per_seq` of them for one sequence, `max_slots` live sequences."""
    n_pages: int
    page_size: int
    max_slots: int
    pages_per_seq: int
    max_context: int
    dtype: torch.dtype
    device: object


class CacheGroup:
    """Storage for the cache entries `entries`.  Every call below comes from the host, before a
    step's kernels are launched or after they are queued; none may wait for the device."""

    entries: list[int]

    def start(self, slot: int) -> None:
        """A sequence starts in `slot`: what the last sequence left there must not show."""

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        """Room for positions [old_len, new_len) of the sequence in `slot`; raises CacheError if there is none
        (before anything of the step is launched)."""

    def commit(self, slot: int, length: int) -> None:
        """The step is queued; the sequence now holds `length` tokens.  What no later token needs may go back."""

    def reserve_one_each(self, slots, old_lens) -> None:
        """reserve(slot, old, old + 1) for many sequences at once (numpy arrays): the step of one token per
        sequence, which a group may do faster than one call per sequence."""
        for slot, old in zip(slots.tolist(), old_lens.tolist()):
            self.reserve(slot, old, old + 1)

    def commit_one_each(self, slots, new_lens) -> None:
        for slot, length in zip(slots.tolist(), new_lens.tolist()):
            self.commit(slot, length)

    def release(self, slot: int) -> None:
        """The sequence in `slot` has ended: everything it holds goes back."""

    def upload(self) -> None:
        """Bring the device's copy of the group's tables up to date (called once before a step's kernels)."""

    def view(self, entry: int):
        """What the mixer of cache entry `entry` is given as `cache_view`."""
        raise NotImplementedError

    def nbytes(self) -> int:
        return 0

    def pages_in_use(self) -> int:
        return 0
