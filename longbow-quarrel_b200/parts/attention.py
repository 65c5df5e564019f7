"""Grouped-query causal attention over the cache.

Order of work as in the reference's block (internal/device/metal.go:1377-1435):
q, k, v projections without bias; position encoding on q and k; k and v stored in
the cache at the token's position; for each query head h the keys of kv head
h // (H / Hkv) from `start` to the token's own position, scores q.k * scale,
softmax, weighted sum of v (internal/device/kernels.metal:657-766); output
projection added to the residual stream.  `window` w restricts the keys to the
last w positions (start = p - w + 1, internal/device/kernels.metal:676).

The three projections are one matrix product over the concatenated weight
[(H + 2 Hkv) hd, D]; rotation and cache write are one kernel.
"""
from __future__ import annotations

import torch

from ..kernels import attention as attention_kernels
from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import KVNeed, Mixer, Runtime, StepContext
from .registry import make_part, register_part
from .spec import PartSpec

DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True
    folds_norm = True

    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position: PartSpec | None = None, window: int | None = None,
                 own_kv: bool = True, names: dict | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 2 or not 2 <= head_dim <= 256:
            # Pairs of the rotation need an even size; the plain kernels hold a head in 256 threads' registers.
            # Which of the faster kernels take a head size is each kernel's own rule (kernels/attention.py).
            raise ValueError(f"attention: head_dim {head_dim} must be even and at most 256")
        self.runtime = runtime
        self.D, self.H, self.Hkv, self.hd = hidden_size, n_heads, n_kv_heads, head_dim
        self.scale, self.window, self.own_kv = float(scale), window, own_kv
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.position = make_part("position", position, runtime) if position is not None else None
        self.w_qkv: linear.LinearWeight | None = None
        self.w_o: linear.LinearWeight | None = None

    def cache_need(self):
        return KVNeed(self.Hkv, self.hd, self.window)

    def step_needs(self):
        return attention_kernels.step_needs(self.runtime.act_dtype, self.hd, self.H, self.Hkv, self.window,
                                            self.runtime.device)

    def weights(self):
        n = self.names
        out = {n["q"]: WeightSpec((self.H * self.hd, self.D)), n["o"]: WeightSpec((self.D, self.H * self.hd))}
        if self.own_kv:
            out[n["k"]] = WeightSpec((self.Hkv * self.hd, self.D))
            out[n["v"]] = WeightSpec((self.Hkv * self.hd, self.D))
        if self.position is not None:
            out.update(self.position.weights())        # a position encoding may have tensors of its own
        return out

    def load(self, tensors):
        n = self.names
        rows = [tensors[n["q"]]] + ([tensors[n["k"]], tensors[n["v"]]] if self.own_kv else [])
        self.w_qkv = linear.LinearWeight(torch.cat(rows, dim=0))
        self.w_o = linear.LinearWeight(tensors[n["o"]])
        if self.position is not None and self.position.weights():
            self.position.load({name: tensors[name] for name in self.position.weights()})

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True, emit=None):
        store = self.own_kv and writes_cache
        tables = self.position.tables() if self.position is not None else None
        fused = (store and h.dtype == torch.bfloat16 and self.w_qkv.tensor.dtype == torch.bfloat16 and self.D % 8 == 0
                 and self.hd % 16 == 0 and cache_view.k_pages.dtype == torch.bfloat16 and (self.position is None or tables is not None))
        few = h.shape[0] <= 16 and ops.streams_through_registers(h.shape[0], self.w_qkv.N)
        if fused and (few or (self.hd in (64, 128) and not isinstance(h, ops.NormedRows))):
            # Projection, rotation and cache write are one kernel (for few tokens the one that streams the
            # weights through registers, else the tcgen05 one).
            cos, sin = tables if tables is not None else (None, None)
            linear.note(self.w_qkv)
            qkv_kernel = ops.gemm_skinny_qkv if few else ops.gemm_tc_qkv
            q = qkv_kernel(h, self.w_qkv.tensor, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                           cache_view.page_table, cache_view.k_pages, cache_view.v_pages, self.H, self.Hkv,
                           self.hd, cache_view.page_size)
            out = attention_kernels.attention(q, cache_view, ctx, self.H, self.Hkv, self.hd, self.scale, self.window,
                                              next_w=self.w_o.tensor)
            return self._project(out, residual, emit)
        qkv = linear.linear(h, self.w_qkv, self.runtime.act_dtype)
        if self.position is not None and tables is None:
            q = qkv[:, :self.H * self.hd].unflatten(1, (self.H, self.hd))
            k = qkv[:, self.H * self.hd:(self.H + self.Hkv) * self.hd].unflatten(1, (self.Hkv, self.hd)) \
                if self.own_kv else None
            self.position.apply(q, k, ctx.tok_pos)
        cos, sin = tables if tables is not None else (None, None)
        if not self.own_kv:
            ops.rope_kv_write(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots, None, None, None,
                              self.H, self.Hkv, self.hd, cache_view.page_size)
        else:
            if not store:
                raise ValueError("attention: a layer with its own k and v must write its cache entry")
            ops.rope_kv_write(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots, cache_view.page_table,
                              cache_view.k_pages, cache_view.v_pages, self.H, self.Hkv, self.hd, cache_view.page_size)
        out = attention_kernels.attention(qkv, cache_view, ctx, self.H, self.Hkv, self.hd, self.scale, self.window,
                                          next_w=self.w_o.tensor)
        return self._project(out, residual, emit)

    def _project(self, out, residual, emit):
        """Output projection added into the residual; with `emit`, the next norm's rows (or None)."""
        if emit is None:
            linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual)
            return None
        return linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual, emit=emit)[1]
