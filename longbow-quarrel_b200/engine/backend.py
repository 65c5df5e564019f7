"""What the generation loop drives when it runs on the engine: the step function,
then the sampler on the logits, then the sampled ids back to the host."""
from __future__ import annotations

import torch

from ..sampling import SamplingParams, history_window, sample


class EngineBackend:
    def __init__(self, engine, params: SamplingParams):
        self.engine, self.params = engine, params
        self.seed = params.resolved_seed()
        self._scratch = None

    def start(self) -> int:
        return self.engine.new_sequence()

    def finish(self, handle: int) -> None:
        self.engine.end_sequence(handle)

    def run(self, entries, requests, steps, histories) -> list[int]:
        logits = self.engine.stepper.step(entries, None)
        dev = logits.device
        seq_ids = step_ids = hist = hist_len = None
        if not self.params.greedy:
            ids = torch.tensor([requests, steps], dtype=torch.int32).to(dev)
            seq_ids, step_ids = ids[0], ids[1]
        if self.params.uses_history:
            h, n = history_window(histories)
            hist, hist_len = torch.from_numpy(h).to(dev), torch.from_numpy(n).to(dev)
        if self._scratch is None or self._scratch.shape[0] < logits.shape[0]:
            self._scratch = torch.empty_like(logits)
        tokens = sample(logits, self.params, self.seed, seq_ids, step_ids, hist, hist_len,
                        scratch=self._scratch[:logits.shape[0]])
        return tokens.tolist()
