"""The step function: a batch of sequences, each with its next tokens (a whole
prompt, or one token), run as one packed batch from the cache; logits come back
for the wanted rows only.

The reference runs one token of one sequence per layer call
(internal/engine/engine.go:1358-1605) and computes logits for the last prompt
position only (engine.go:1505).  Here rows of all sequences are packed
[T_total, D]; each row knows its sequence and its position, so padding does not
exist and a row's result does not depend on its neighbours.
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache import Cache
from ..kernels import ops
from ..parts.base import StepContext, StepShape


class StepError(ValueError):
    pass


def check_entries(entries, want, vocab_size: int) -> None:
    """Errors that are found before anything is launched (empty input and token
    range as in internal/engine/engine.go:1300,1327-1331)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    seen = set()
    for b, (slot, tokens) in enumerate(entries):
        if slot in seen:
            raise StepError(f"slot {slot} appears twice in one step")
        seen.add(slot)
        if len(tokens) == 0:
            raise StepError(f"sequence {b} of the step brings no tokens")
        for i, t in enumerate(tokens):
            if not 0 <= int(t) < vocab_size:
                raise StepError(f"token {t} at place {i} of sequence {b} is outside the vocabulary [0, {vocab_size})")
    if want is not None:
        if len(want) != len(entries):
            raise StepError("`want` must have one list for each sequence of the step")
        for b, (ws, (_, tokens)) in enumerate(zip(want, entries)):
            for w in ws:
                if not 0 <= int(w) < len(tokens):
                    raise StepError(f"wanted place {w} of sequence {b} is outside its {len(tokens)} tokens")


def pack_step(entries, want, past: list[int], needs: dict | None = None) -> tuple[np.ndarray, dict]:
    """All integers a step's kernels read, in one int32 array, and where each part lies.
    `want` None asks for the last row of every sequence.  `needs`: name -> function of the step's
    shape, for the arrays that parts of the model asked for (`Part.step_needs`)."""
    B = len(entries)
    new = [len(t) for _, t in entries]
    T = sum(new)
    cu = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(new, out=cu[1:])
    tokens = np.concatenate([np.asarray(t, dtype=np.int64) for _, t in entries])
    tok_seq = np.repeat(np.arange(B), new)
    tok_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(past, new)])
    slots = np.asarray([s for s, _ in entries])
    kv_len = np.asarray([p + n for p, n in zip(past, new)])
    if want is None:
        rows = cu[1:] - 1
    else:
        rows = np.asarray([cu[b] + int(w) for b, ws in enumerate(want) for w in ws], dtype=np.int64)
    parts = {"tokens": tokens, "tok_seq": tok_seq, "tok_pos": tok_pos, "slots": slots, "kv_len": kv_len,
             "cu_rows": cu, "want_rows": rows}
    if needs:
        shape = StepShape(B=B, T=T, past=tuple(int(p) for p in past), new=tuple(new), cu=tuple(int(c) for c in cu))
        for name, build in needs.items():
            if name in parts:
                raise StepError(f"a part asks for a step array named {name!r}, which the step context uses itself")
            parts[name] = np.asarray(build(shape)).reshape(-1)
    layout, offset = {}, 0
    for name, arr in parts.items():
        layout[name] = (offset, len(arr))
        offset += -(-len(arr) // 4) * 4  # every part starts on a 16-byte boundary
    flat = np.zeros(max(offset, 4), dtype=np.int32)
    for name, arr in parts.items():
        o, n = layout[name]
        flat[o:o + n] = arr
    info = {"layout": layout, "B": B, "T": T, "new": new, "past": list(past), "max_new": max(new),
            "max_kv": int(kv_len.max()), "extra": [n for n in parts if needs and n in needs]}
    return flat, info


def make_context(flat_dev: torch.Tensor, info: dict, h_slots: list[int]) -> StepContext:
    def part(name):
        o, n = info["layout"][name]
        return flat_dev[o:o + n]
    want = part("want_rows")
    return StepContext(T=info["T"], B=info["B"], tokens=part("tokens"), tok_seq=part("tok_seq"),
                       tok_pos=part("tok_pos"), slots=part("slots"), kv_len=part("kv_len"), cu_rows=part("cu_rows"),
                       want_rows=want if want.numel() else None, h_slots=h_slots, h_new=info["new"],
                       h_past=info["past"], max_new=info["max_new"], max_kv=info["max_kv"],
                       extra={name: part(name) for name in info.get("extra", [])})


class Stepper:
    """Runs steps of one model on one cache.  Steps in which every sequence brings one
    token are captured once per batch size in a CUDA graph and replayed, because such a
    step is a few hundred short kernels whose launches would otherwise cost more than
    their work; all other steps launch their kernels one by one."""

    def __init__(self, model, cache: Cache, device, use_graphs: bool = True):
        self.model, self.cache, self.device = model, cache, device
        self.use_graphs = use_graphs and model.graph_safe
        self.needs = model.step_needs()
        self._graphs: dict[int, "_DecodeGraph"] = {}
        self._seen: set[int] = set()

    def step(self, entries, want=None) -> torch.Tensor | None:
        """entries: [(slot, tokens)], want: [[places]] or None (= each sequence's last token).
        Returns logits [n_wanted, vocab] float32 in the order of entries and of want."""
        check_entries(entries, want, self.model.spec.vocab_size)
        if all(len(t) == 1 for _, t in entries) and self._replays(len(entries)):
            logits = self._replay_step([s for s, _ in entries], [int(t[0]) for _, t in entries], None)
            return self._wanted(logits, want, len(entries))
        past = [self.cache.length(slot) for slot, _ in entries]
        for slot, tokens in entries:
            self.cache.reserve(slot, len(tokens))
        self.cache.upload()
        decode = all(len(t) == 1 for _, t in entries)
        if decode and self.use_graphs and self.model.probe is None:
            logits = self._decode_step(entries, want, past)
        else:
            flat, info = pack_step(entries, want, past, self.needs)
            flat_dev = torch.from_numpy(flat).to(self.device)
            ctx = make_context(flat_dev, info, [s for s, _ in entries])
            logits = self.model.forward(ctx, self.cache)
        for slot, tokens in entries:
            self.cache.commit(slot, len(tokens))
        return logits

    def step_fed(self, slots: list[int], source: torch.Tensor, rows: list[int] | None = None) -> torch.Tensor:
        """One more token for each sequence in `slots`, the tokens taken on the device from
        `source` (int32, e.g. what the sampler wrote for the step before): sequence b gets
        source[rows[b]] (source[b] without rows).  The host never sees these tokens before the
        step is launched, so the step can be queued while the one before it still runs."""
        if rows is not None and rows != list(range(len(rows))):
            source = source[torch.tensor(rows, dtype=torch.long, device=self.device)]
        elif source.numel() != len(slots):
            source = source[:len(slots)]
        if self._replays(len(slots)):
            return self._replay_step(slots, None, source)
        entries = [(s, [0]) for s in slots]
        past = [self.cache.length(s) for s in slots]
        for s in slots:
            self.cache.reserve(s, 1)
        self.cache.upload()
        if self.use_graphs and self.model.probe is None:
            logits = self._decode_step(entries, None, past, fed=source)
        else:
            flat, info = pack_step(entries, None, past, self.needs)
            flat_dev = torch.from_numpy(flat).to(self.device)
            ctx = make_context(flat_dev, info, slots)
            ctx.tokens.copy_(source)
            logits = self.model.forward(ctx, self.cache)
        for s in slots:
            self.cache.commit(s, 1)
        return logits

    # ------------------------------------------------------------------ steps of one token per sequence
    def _replays(self, B: int) -> bool:
        """Whether a step of one token for each of B sequences is a replay of a captured step."""
        return self.use_graphs and self.model.probe is None and B in self._graphs

    def _replay_step(self, slots: list[int], tokens: list[int] | None, fed: torch.Tensor | None) -> torch.Tensor:
        """The step that generation repeats most, with as little host work as it needs: the cache's
        bookkeeping for all sequences at once, the step's integers written into the captured step's layout
        (what never changes between steps is there already), one copy, one replay."""
        graph = self._graphs[len(slots)]
        past = self.cache.reserve_one_each(slots)
        self.cache.upload()
        logits = graph.replay(graph.fill(slots, tokens, past, self.needs), fed)
        self.cache.commit_one_each(slots)
        return logits

    def _wanted(self, logits, want, B: int):
        if want is None:
            return logits
        rows = [b for b, ws in enumerate(want) for _ in ws]
        if rows == list(range(B)):
            return logits
        if not rows:
            return None
        return logits[torch.tensor(rows, device=self.device)]

    def _decode_step(self, entries, want, past, fed: torch.Tensor | None = None):
        B = len(entries)
        flat, info = pack_step(entries, None, past, self.needs)
        if B not in self._seen:
            # The first step of a batch size runs eagerly: it loads kernels and sizes buffers.
            self._seen.add(B)
            flat_dev = torch.from_numpy(flat).to(self.device)
            ctx = make_context(flat_dev, info, [s for s, _ in entries])
            if fed is not None:
                ctx.tokens.copy_(fed)
            logits = self.model.forward(ctx, self.cache)
        else:
            graph = self._graphs.get(B)
            if graph is None:
                graph = self._graphs[B] = _DecodeGraph(self.model, self.cache, self.device, flat, info)
            logits = graph.replay(flat, fed)
        return self._wanted(logits, want, B)


class _DecodeGraph:
    """One captured step for a batch of B sequences with one token each.  The integers
    of a step (tokens, positions, slots) are copied into the buffer the graph reads."""

    def __init__(self, model, cache, device, flat: np.ndarray, info: dict):
        self.device = device
        self.host = torch.empty(len(flat), dtype=torch.int32).pin_memory()
        self.flat_dev = torch.zeros(len(flat), dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event()
        self.info = dict(info)
        # Kernels that size their work by the longest sequence are captured for the longest possible one.
        self.info["max_kv"] = cache.max_context
        self.template = np.array(flat, dtype=np.int32)          # a step's integers in this layout, filled anew each step
        self.host.numpy()[:] = flat
        self.flat_dev.copy_(self.host, non_blocking=True)
        ctx = make_context(self.flat_dev, self.info, list(range(info["B"])))
        self.graph = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream(device))
        before, names = ops.launch_count(), ops.launches_by_name()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(self.graph, stream=stream):
                self.logits = model.forward(ctx, cache)
        self.kernels, self.by_name = ops.launch_count() - before, ops.launches_since(names)
        ops.add_launches(-self.kernels, self.by_name, -1)      # recorded, not run
        torch.cuda.current_stream(device).wait_stream(stream)
        self.copied.record()

    def fill(self, slots: list[int], tokens: list[int] | None, past: np.ndarray, needs: dict) -> np.ndarray:
        """The integers of a step of one token per sequence, in this graph's layout.  Which row belongs to
        which sequence, where the rows start and which rows are wanted is the same in every such step and stays
        as the capture left it; tokens, slots, positions and lengths are written anew, and so are the arrays
        that parts asked for, where they are not empty."""
        flat, layout = self.template, self.info["layout"]
        if tokens is not None:
            o, n = layout["tokens"]
            flat[o:o + n] = tokens
        o, n = layout["slots"]
        flat[o:o + n] = slots
        o, n = layout["tok_pos"]
        flat[o:o + n] = past
        o, n = layout["kv_len"]
        flat[o:o + n] = past + 1
        for name in self.info["extra"]:
            o, n = layout[name]
            if n:
                B = len(slots)
                flat[o:o + n] = np.asarray(needs[name](StepShape(B=B, T=B, past=tuple(past.tolist()), new=(1,) * B,
                                                                 cu=tuple(range(B + 1))))).reshape(-1)
        return flat

    def replay(self, flat: np.ndarray, fed: torch.Tensor | None = None) -> torch.Tensor:
        self.copied.synchronize()
        self.host.numpy()[:] = flat
        self.flat_dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        if fed is not None:
            o, n = self.info["layout"]["tokens"]
            self.flat_dev[o:o + n].copy_(fed)
        self.graph.replay()
        ops.add_launches(self.kernels, self.by_name)
        return self.logits
