"""A model built from its description: embedding, blocks, the order they run in,
final norm, head.  It owns the parts and their weights; it owns no cache."""
from __future__ import annotations

import torch

from ..kernels import linear
from ..parts.base import Runtime, StepContext
from ..parts.registry import make_part
from ..parts.spec import ModelSpec, PartSpec
from ..weights.spec import WeightSpec


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.embedding = make_part("embedding", spec.embedding, runtime)
        self.blocks = [make_part("block", PartSpec(layer.arrangement), runtime, layer=layer) for layer in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm, runtime)
        self.head = make_part("head", spec.head, runtime)
        self._order_known = False
        # probe(run, x, ctx): called with the residual stream after the embedding (run -1) and after every
        # scheduled run of a layer, for looking into a step (trace replay's per-layer statistics).  Steps
        # with a probe are not replayed from CUDA graphs.
        self.probe = None
        for n, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {n} names layer {entry.layer}; the model has {len(self.blocks)}")
        writers = [e.cache for e in spec.schedule if e.writes_cache]
        if len(set(writers)) != len(writers):
            raise ValueError("schedule: two runs write the same cache entry")
        for e in spec.schedule:
            if not e.writes_cache and e.cache not in writers:
                raise ValueError(f"schedule: a run reads cache entry {e.cache}, which no run writes")

    # ------------------------------------------------------------------ weights
    def _named_parts(self):
        yield "", self.embedding
        for block in self.blocks:
            yield block.prefix, block
        yield "", self.final_norm
        yield "", self.head

    def weight_table(self) -> dict[str, WeightSpec]:
        """Every tensor the model reads, by its full name."""
        table: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for name, spec in part.weights().items():
                full = prefix + name
                if full in table:
                    raise ValueError(f"two parts name the tensor {full!r}")
                table[full] = spec
        return table

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self._named_parts():
            mine = {}
            for name, spec in part.weights().items():
                if prefix + name in tensors:
                    mine[name] = tensors[prefix + name]
                elif spec.fallback is None:
                    raise KeyError(prefix + name)
            for full in part.borrows():              # tensors of other parts that this one reads as well
                if full in tensors:
                    mine[full] = tensors[full]
            part.load(mine)

    @property
    def graph_safe(self) -> bool:
        """Every part allows its steps to be captured in a CUDA graph."""
        return all(part.graph_safe for _, part in self._named_parts())

    def cache_needs(self) -> dict:
        """Cache entry -> what the mixer that writes it needs."""
        return {e.cache: self.blocks[e.layer].cache_need() for e in self.spec.schedule if e.writes_cache}

    def step_needs(self) -> dict:
        """Name -> builder of every per-step integer array that some part asks for (see Part.step_needs)."""
        out = {}
        for _, part in self._named_parts():
            out.update(part.step_needs())
        return out

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for _, part in self._named_parts():
            for t in _tensors_of(part):
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, cache) -> torch.Tensor | None:
        """Run this step's rows through every scheduled layer; logits [wanted, vocab]
        (float32) at ctx.want_rows, or None when nothing is wanted."""
        if not self._order_known:
            # The first step also notes in which order the weights are read (it is the same in every step).
            self._order_known = True
            with linear.recording():
                return self.forward(ctx, cache)
        x = self.embedding.forward(ctx.tokens)
        schedule = self.spec.schedule
        probe = self.probe
        if probe is not None:
            probe(-1, x, ctx)
        normed = None           # rows of the next layer's first norm, when this layer's last product made them
        for i, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if not getattr(block, "folds_norm", False):
                block.forward(x, ctx, cache.view(entry.cache), entry.writes_cache)
                normed = None
                if probe is not None:
                    probe(i, x, ctx)
                continue
            after = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            emit = after.input_norm(x.shape[0]) if getattr(after, "folds_norm", False) else None
            normed = block.forward(x, ctx, cache.view(entry.cache), entry.writes_cache, normed=normed, emit=emit)
            if probe is not None:
                probe(i, x, ctx)
        if ctx.want_rows is None or ctx.want_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, rows=ctx.want_rows)
        return self.head.forward(h)


def _tensors_of(obj, depth: int = 0):
    if depth > 3:
        return
    for value in vars(obj).values():
        if isinstance(value, torch.Tensor):
            yield value
        elif hasattr(value, "tensor") and isinstance(getattr(value, "tensor"), torch.Tensor):
            yield value.tensor
        elif hasattr(value, "__dict__") and not isinstance(value, (Runtime, type)) and hasattr(value, "weights"):
            yield from _tensors_of(value, depth + 1)
