"""The arrangement of parts in a layer.

"pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x)), the order of the reference's
block (internal/device/metal.go:1347-1527), with the residual stream x in 32-bit
throughout (internal/engine/engine.go:1375)."""
from __future__ import annotations

from .base import Part, Runtime, StepContext
from .registry import make_part, register_part
from .spec import LayerSpec


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    def __init__(self, runtime: Runtime, layer: LayerSpec):
        self.prefix = layer.prefix
        unknown = set(layer.parts) - {"norm1", "mixer", "norm2", "ffn"}
        if unknown:
            raise ValueError(f"layer {layer.prefix!r}: the arrangement 'pre_norm' has no place {sorted(unknown)}")
        self.norm1 = make_part("norm", layer.part("norm1"), runtime)
        self.mixer = make_part("mixer", layer.part("mixer"), runtime)
        self.norm2 = make_part("norm", layer.part("norm2"), runtime)
        self.ffn = make_part("ffn", layer.part("ffn"), runtime)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def cache_need(self):
        """What the layer's cache entry must hold: its mixer's need."""
        return self.mixer.cache_need()

    def step_needs(self):
        out = {}
        for part in self.parts():
            out.update(part.step_needs())
        return out

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def weights(self):
        out = {}
        for part in self.parts():
            for name, spec in part.weights().items():
                if name in out:
                    raise ValueError(f"layer {self.prefix}: two parts name the tensor {name!r}")
                out[name] = spec
        return out

    def load(self, tensors):
        for part in self.parts():
            part.load({n: tensors[n] for n in part.weights()})

    folds_norm = True

    def input_norm(self, n_rows: int):
        """(gain, eps) when the layer ahead of this one may leave this layer's first norm to the
        products on either side of it; None otherwise."""
        return self.norm1.foldable(n_rows) if self.mixer.folds_norm else None

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool = True, normed=None, emit=None):
        """`normed`: the rows of norm1, when the layer ahead made them (see input_norm).  `emit`: the
        input_norm() of the layer that follows.  Returns that layer's rows, or None."""
        n_rows = x.shape[0]
        h = normed if normed is not None else self.norm1.forward(x)
        fold2 = self.norm2.foldable(n_rows) if (self.mixer.folds_norm and self.ffn.folds_norm) else None
        h = self.mixer.forward(h, ctx, cache_view, x, writes_cache, emit=fold2) if fold2 is not None \
            else self.mixer.forward(h, ctx, cache_view, x, writes_cache)
        if fold2 is None or h is None:
            h = self.norm2.forward(x)
        if emit is not None and self.ffn.folds_norm:
            return self.ffn.forward(h, ctx, x, emit=emit)
        self.ffn.forward(h, ctx, x)
        return None
