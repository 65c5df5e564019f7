"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier, and as many batches one after another as there are requests.

The reference generates for one sequence: a prefill loop, the first token sampled
from the last prompt position, then a decode loop that stops at the end-of-text id
without returning it (internal/engine/engine.go:1358-1762, the stop at :1744).
The loop here decides the same things for a batch; it knows nothing of the GPU and
talks to a backend, so its decisions are tested with a scripted one.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Protocol, Sequence


class Backend(Protocol):
    # A backend whose sampling never looks at the tokens so far may set `needs_history = False`; `run` is then
    # given None for `histories` (building them costs time in every step of a long generation).
    def start(self) -> int: ...
    def finish(self, handle: int) -> None: ...
    def run(self, entries: list[tuple[int, list[int]]], requests: list[int], steps: list[int],
            histories: list[list[int]]) -> list[int]: ...


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0
    finish_reasons: list[str] = field(default_factory=list)

    @property
    def decode_tokens_per_second(self) -> float:
        n = self.generated_tokens - len(self.finish_reasons)
        return n / self.decode_seconds if self.decode_seconds > 0 and n > 0 else 0.0


def generate(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int, stop_ids: Sequence[int] = (),
             callback: Callable[[int, int], None] | None = None, include_stop: bool = False,
             batch_size: int = 64, max_context: int | None = None) -> tuple[list[list[int]], GenerationStats]:
    """Returns the new tokens of every prompt, in the order of the prompts."""
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")  # "empty input tokens", internal/engine/engine.go:1300
        if max_context is not None and len(p) > max_context:
            raise ValueError(f"prompt {i} has {len(p)} tokens; the context limit is {max_context}")
    if batch_size < 1:
        raise ValueError("batch_size must be at least 1")
    stops = set(int(s) for s in stop_ids)
    with_history = getattr(backend, "needs_history", True)
    outputs: list[list[int]] = [[] for _ in prompts]
    stats = GenerationStats(finish_reasons=["" for _ in prompts])
    if max_new_tokens <= 0:
        stats.finish_reasons = ["length" for _ in prompts]
        return outputs, stats

    for b0 in range(0, len(prompts), batch_size):
        batch = list(range(b0, min(len(prompts), b0 + batch_size)))
        handles = {i: backend.start() for i in batch}
        live = list(batch)
        stats.batches += 1
        try:
            t0 = time.perf_counter()
            sampled = backend.run([(handles[i], list(prompts[i])) for i in live], live, [0] * len(live),
                                  [list(prompts[i]) for i in live] if with_history else None)
            stats.prefill_seconds += time.perf_counter() - t0
            stats.prompt_tokens += sum(len(prompts[i]) for i in live)
            step = 0
            while True:
                still = []
                for i, tok in zip(live, sampled):
                    tok = int(tok)
                    reason = ""
                    if tok in stops:
                        reason = "stop"
                        if include_stop:
                            outputs[i].append(tok)
                    else:
                        outputs[i].append(tok)
                        if callback is not None:
                            callback(i, tok)
                        if len(outputs[i]) >= max_new_tokens:
                            reason = "length"
                        elif max_context is not None and len(prompts[i]) + len(outputs[i]) >= max_context:
                            reason = "context"
                    if reason:
                        stats.finish_reasons[i] = reason
                        backend.finish(handles.pop(i))   # the sequence ends: its slot and pages go back now
                    else:
                        still.append(i)
                stats.generated_tokens += len(live)
                live = still
                if not live:
                    break
                step += 1
                t0 = time.perf_counter()
                sampled = backend.run([(handles[i], [outputs[i][-1]]) for i in live], live, [step] * len(live),
                                      [list(prompts[i]) + outputs[i] for i in live] if with_history else None)
                stats.decode_seconds += time.perf_counter() - t0
                stats.decode_steps += 1
        finally:
            for h in handles.values():
                backend.finish(h)
    return outputs, stats
