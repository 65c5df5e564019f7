"""What every part is: sizes and constants given at construction, the tensors it
needs, and a forward that works on the packed rows of one step.

The runtime says where and in which precision a model runs; the step context says
which rows belong to which sequence and where they stand.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import numpy as np
import torch

from ..weights.spec import WeightSpec


@dataclass
class Runtime:
    """Where a model runs.  dtype float32 = every tensor and product in true 32-bit;
    bfloat16 = bfloat16 weights, activations and cache with a 32-bit residual stream,
    32-bit norms, softmax, rotation and accumulation."""
    device: torch.device
    dtype: torch.dtype
    max_context: int
    shared: dict = field(default_factory=dict)  # tables shared by equal parts (rope cos/sin)

    @property
    def act_dtype(self) -> torch.dtype:
        return self.dtype


@dataclass(frozen=True)
class StepShape:
    """What the host knows of a step before it is packed: for each of its B sequences how many tokens
    it holds already (`past`) and how many it brings (`new`), and where each sequence's rows start in
    the packed batch (`cu`, B + 1 entries).  Parts build their own per-step integers from it."""
    B: int
    T: int
    past: tuple[int, ...]
    new: tuple[int, ...]
    cu: tuple[int, ...]

    @property
    def max_new(self) -> int:
        return max(self.new)


@dataclass
class StepContext:
    """The packed rows of one step.  T rows of B sequences; row r belongs to sequence
    tok_seq[r] of the batch and stands at position tok_pos[r] of that sequence; the
    sequence lives in cache slot slots[b] and holds kv_len[b] tokens once this step's
    rows are stored.  All tensors are int32 on the device; the `h_` twins are host lists.
    `extra` holds the int32 arrays that parts asked for through `Part.step_needs`, by name."""
    T: int
    B: int
    tokens: torch.Tensor
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    slots: torch.Tensor
    kv_len: torch.Tensor
    cu_rows: torch.Tensor
    want_rows: torch.Tensor | None
    h_slots: list[int]
    h_new: list[int]
    h_past: list[int]
    max_new: int
    max_kv: int
    extra: dict = field(default_factory=dict)

    @property
    def decode(self) -> bool:
        return self.max_new == 1


class Part:
    """Base of all parts.

    graph_safe: the part's forward launches the same work for every step of a batch
    size and reads positions, slots and lengths from the step context's device tensors
    only, so a step that contains it may be captured in a CUDA graph and replayed.  A
    part that looks at the context's host lists must leave this False."""

    graph_safe = False

    def weights(self) -> dict[str, WeightSpec]:
        """Tensor name (relative to the part's prefix) -> what it must look like."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Take the tensors named by weights() (already on the device)."""

    def borrows(self) -> list[str]:
        """Full names of tensors of other parts that this part reads as well (a head tied to the
        embedding table); `load` is given them beside its own."""
        return []

    def step_needs(self) -> dict[str, Callable[[StepShape], np.ndarray]]:
        """Integers that this part's kernels need for every step beyond the step context's own fields: a
        name, and a function that makes the array from the step's shape on the host.  The step function
        packs every array that some part of the model names (once per name) into the step's one buffer
        and hands it over as `ctx.extra[name]` (int32, on the device).  For steps of one token per
        sequence the array's length may depend on the number of sequences only (such steps are captured
        once per batch size)."""
        return {}


class CacheNeed:
    """What a mixer asks of the cache for one cache entry.  Entries whose needs are equal (needs are
    hashable values) share one group of storage; the need itself says which kind of group that is, so a
    mixer with storage of another shape brings its own: a frozen dataclass derived from this, whose
    `make_group` returns a `cache.group.CacheGroup`."""

    def make_group(self, entries: list[int], sizing):
        """Storage for the cache entries `entries` (all with this need).  `sizing` is a
        `cache.group.CacheSizing`: pages, page size, slots, dtype, device."""
        raise NotImplementedError


@dataclass(frozen=True)
class KVNeed(CacheNeed):
    """A mixer that keeps keys and values of every position (or of the last `window`)."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None

    def make_group(self, entries, sizing):
        from ..cache.paged import PagedKVGroup
        return PagedKVGroup(entries, self.n_kv_heads, self.head_dim, self.window, sizing.n_pages, sizing.page_size,
                            sizing.max_slots, sizing.pages_per_seq, sizing.dtype, sizing.device)


@dataclass(frozen=True)
class StateNeed(CacheNeed):
    """A mixer that keeps a state of fixed size for each sequence."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def make_group(self, entries, sizing):
        from ..cache.state import StateGroup
        return StateGroup(entries, self.shape, self.dtype, sizing.max_slots, sizing.device)


class Mixer(Part):
    # A part that sets this takes unfinished rows of a norm (kernels.ops.NormedRows) as `h` and takes
    # the keyword `emit`: (gain, eps) of the RMS norm that reads the residual next.  With `emit` it
    # returns that norm's rows, made in the epilogue of its last product, or None where it cannot.
    # A part that leaves it False is always given finished rows and its return value is not read.
    folds_norm = False

    def cache_need(self) -> CacheNeed | None:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache_view, residual: torch.Tensor,
                writes_cache: bool = True) -> None:
        """Read the normed rows h [T, D]; add the mixer's output to residual [T, D] (float32)."""
        raise NotImplementedError


class FeedForward(Part):
    folds_norm = False        # as for Mixer

    def forward(self, h: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        """Read the normed rows h [T, D]; add the output to residual [T, D] (float32)."""
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """Normalise rows of the float32 stream; returns the activation dtype."""
        raise NotImplementedError

    def foldable(self, n_rows: int) -> tuple | None:
        """(gain, eps) when this norm is x / rms(x) * gain and the products on either side of it can
        do its work for `n_rows` rows (see Mixer.folds_norm); None otherwise."""
        return None


class PositionEncoding(Part):
    """Either gives cos/sin tables for the fused rotate-and-store kernel, or rotates
    q and k itself in `apply` (then `tables` returns None)."""

    def tables(self) -> tuple[torch.Tensor, torch.Tensor] | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor | None, positions: torch.Tensor) -> None:
        """Rotate q [T, H, hd] and k [T, Hkv, hd] in place."""
