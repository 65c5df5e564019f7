"""Per-sequence state of fixed size, one record per slot and cache entry.

The reference keeps such state for its recurrent layers ([dConv, k] and
[dInner, dState] per layer, internal/engine/mamba.go:102-114) and one cache
position for its single sequence (internal/engine/types.go:218).  Llama 3's
attention needs none, but the storage is part of the cache so that a mixer that
does gets a zeroed record when its sequence starts."""
from __future__ import annotations

import torch

from .group import CacheGroup


class StateGroup(CacheGroup):
    def __init__(self, entries: list[int], shape: tuple[int, ...], dtype: torch.dtype, max_slots: int, device):
        self.entries = list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.shape, self.dtype = tuple(shape), dtype
        self.data = torch.zeros((len(self.entries), max_slots, *self.shape), dtype=dtype, device=device)

    def start(self, slot: int) -> None:
        self.data[:, slot].zero_()

    reset = start

    def reserve_one_each(self, slots, old_lens) -> None:
        pass

    def commit_one_each(self, slots, new_lens) -> None:
        pass

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def view(self, entry: int) -> torch.Tensor:
        """[max_slots, *shape] of one cache entry."""
        return self.data[self.index[entry]]
