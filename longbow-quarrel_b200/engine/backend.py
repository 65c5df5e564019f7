"""What the generation loop drives when it runs on the engine: the step function,
then the sampler on the logits, then the sampled ids back to the host.

The loop asks for one step at a time and needs the sampled ids on the host to decide
who stops.  So that the GPU does not idle while the host decides and prepares, the backend
queues the step after the one asked for before it hands the ids back: that step takes its
tokens on the device, straight from the sampler's output, and assumes that every sequence
goes on.  When the loop then asks for that step, its work is already running; a sequence
that stopped meanwhile has cost one unused row.  Sampling that needs the token history on
the host (a repetition penalty) does not run ahead.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache import CacheError
from ..kernels import ops
from ..sampling import SamplingParams, history_window, sample
from ..sampling.sampler import needs_scratch


@dataclass
class _Sampled:
    """The sampled ids of one step: on the device, and on their way to pinned host memory (the
    copy is queued right behind the sampler, before any later step, so that waiting for it does
    not wait for a step that was queued ahead)."""
    handles: tuple[int, ...]
    asked: tuple                  # (handle, request, step) of each row: which step of which request this is
    device: torch.Tensor          # int32 [len(handles)]
    host: torch.Tensor            # pinned int32 [>= len(handles)]
    ready: torch.cuda.Event

    def ids(self) -> list[int]:
        self.ready.synchronize()
        ops.check_status()          # a kernel whose bounded wait gave up left garbage: say so
        return self.host[:len(self.handles)].tolist()


class EngineBackend:
    def __init__(self, engine, params: SamplingParams, run_ahead: bool = True, logits_callback=None):
        """logits_callback(request, step, logits): called with the float32 logits (a host tensor [vocab]) from
        which each token was sampled, before the token is handed back; asking for them costs a copy of every
        step's logits to the host and switches running ahead off (the step queued ahead would overwrite the
        captured step's logits before they are read)."""
        self.engine, self.params = engine, params
        self.seed = params.resolved_seed()
        self.logits_callback = logits_callback
        self.run_ahead = run_ahead and not params.uses_history and logits_callback is None
        self.needs_history = params.uses_history        # the generation loop builds histories only for a penalty
        self._draw_ids: dict = {}                        # requests of a step -> their ids on the device (and zeros)
        self._scratch = None
        self._ahead: _Sampled | None = None
        self._pinned: list[torch.Tensor] = []      # a small ring of pinned buffers for the sampled ids
        self._turn = 0

    def start(self) -> int:
        return self.engine.new_sequence()

    def finish(self, handle: int) -> None:
        self.engine.end_sequence(handle)

    # ------------------------------------------------------------------ one step and its sampling
    def _sample(self, logits, requests, steps, histories):
        dev = logits.device
        seq_ids = step_ids = hist = hist_len = None
        offset = 0
        if not self.params.greedy:
            if len(set(steps)) == 1:
                # The rows advance together (every step of a batch): their ids go to the device once, the step
                # is passed by value.
                key = tuple(requests)
                if key not in self._draw_ids:
                    if len(self._draw_ids) > 64:
                        self._draw_ids.clear()
                    self._draw_ids[key] = torch.tensor([requests, [0] * len(requests)], dtype=torch.int32).to(dev)
                seq_ids, step_ids = self._draw_ids[key]
                offset = int(steps[0])
            else:
                ids = torch.tensor([requests, steps], dtype=torch.int32).to(dev)
                seq_ids, step_ids = ids[0], ids[1]
        if self.params.uses_history:
            h, n = history_window(histories)
            hist, hist_len = torch.from_numpy(h).to(dev), torch.from_numpy(n).to(dev)
        scratch = None
        if needs_scratch(logits.shape[1]):
            if self._scratch is None or self._scratch.shape[0] < logits.shape[0]:
                self._scratch = torch.empty_like(logits)
            scratch = self._scratch[:logits.shape[0]]
        tokens = sample(logits, self.params, self.seed, seq_ids, step_ids, hist, hist_len, scratch=scratch,
                        step_offset=offset)
        n = tokens.numel()
        if len(self._pinned) < 4:
            self._pinned.append(torch.empty(max(n, self.engine.cache.max_slots), dtype=torch.int32).pin_memory())
        self._turn = (self._turn + 1) % 4
        host = self._pinned[min(self._turn, len(self._pinned) - 1)]
        if host.numel() < n:
            host = self._pinned[min(self._turn, len(self._pinned) - 1)] = torch.empty(n, dtype=torch.int32).pin_memory()
        host[:n].copy_(tokens, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record()
        return tokens, host, ready

    def run(self, entries, requests, steps, histories) -> list[int]:
        handles = tuple(h for h, _ in entries)
        asked = tuple(zip(handles, requests, steps))
        ahead, self._ahead = self._ahead, None
        single = all(len(t) == 1 for _, t in entries)
        # The step queued during the last call serves this one only if it is this very step of these very
        # requests.  Handles alone do not say so: a slot that was given back is handed out again, and a new
        # request in it that starts with a one-token prompt looks like the old one going on.
        if ahead is not None and single and set(asked) <= set(ahead.asked):
            current, rows = ahead, [ahead.asked.index(a) for a in asked]
        else:
            if ahead is not None:
                queued = {(h, r) for h, r, _ in ahead.asked}
                wrong = [r for h, r, _ in asked if (h, r) in queued]
                if wrong:
                    # The queued step already stored a token for these requests; it cannot be taken back.
                    raise RuntimeError(f"requests {wrong}: the step after the last one was queued ahead, and another "
                                       f"step is asked for; a backend that runs ahead takes the steps in order")
            logits = self.engine.stepper.step(entries, None)
            current = _Sampled(handles, asked, *self._sample(logits, requests, steps, histories))
            rows = list(range(len(handles)))
            if self.logits_callback is not None:
                host = logits.to("cpu")
                for row, (request, step) in enumerate(zip(requests, steps)):
                    self.logits_callback(request, step, host[row])
        if self.run_ahead:
            try:
                logits = self.engine.stepper.step_fed(list(handles), current.device, rows)
                after = [s + 1 for s in steps]
                self._ahead = _Sampled(handles, tuple(zip(handles, requests, after)),
                                       *self._sample(logits, requests, after, None))
            except CacheError:
                self._ahead = None       # no room for one more token: the loop will end these sequences or fail itself
        ids = current.ids()
        return [ids[r] for r in rows]
