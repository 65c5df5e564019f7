"""Building traces for bin/trace_run, running it, and reading what it wrote."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


def round64(n: int) -> int:
    return -(-n // 64) * 64


class Trace:
    """Steps for trace_run plus, for every wanted row, which (request, position) it is."""

    def __init__(self):
        self.steps: list[dict] = []
        self.rows: dict[int, list[tuple[str, int]]] = {}
        self.max_tokens = 0
        self._live: dict[str, int] = {}

    def add(self, entries: list[tuple[str, list[int], list[int]]], end: list[str] = ()):
        """entries: (request id, tokens, wanted places among them)."""
        step = len(self.steps)
        rows = []
        for rid, tokens, want in entries:
            start = self._live.get(rid, 0)
            self._live[rid] = start + len(tokens)
            rows += [(rid, start + w) for w in want]
        self.max_tokens = max(self.max_tokens, sum(round64(n) for n in self._live.values()))
        self.steps.append({"step": step, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries],
                           "end": list(end)})
        if rows:
            self.rows[step] = rows
        for rid in end:
            del self._live[rid]


def trace_whole(requests: dict[str, list[int]]) -> Trace:
    """Each request alone, all of its tokens in one step, logits everywhere."""
    tr = Trace()
    for rid, tokens in requests.items():
        tr.add([(rid, tokens, list(range(len(tokens))))], end=[rid])
    return tr


def trace_last_one_by_one(requests: dict[str, list[int]], n_last: int = 32) -> Trace:
    """Each request alone: all but the last n_last tokens in one step, then one token a step."""
    tr = Trace()
    for rid, tokens in requests.items():
        head = len(tokens) - n_last
        assert head >= 1
        tr.add([(rid, tokens[:head], [head - 1])])
        for i in range(head, len(tokens)):
            tr.add([(rid, [tokens[i]], [0])], end=[rid] if i == len(tokens) - 1 else [])
    return tr


def trace_batches(requests: dict[str, list[int]], prompt_len: dict[str, int], width: int) -> Trace:
    """Batches of `width` requests that start together with unequal prompts, then go on
    one token each; a request that runs out of tokens ends, the others go on; when a
    batch is over the next one starts (in the slots that were given back)."""
    tr = Trace()
    ids = list(requests)
    for b0 in range(0, len(ids), width):
        batch = ids[b0:b0 + width]
        done = {r: prompt_len[r] for r in batch}
        ends = [r for r in batch if done[r] == len(requests[r])]
        tr.add([(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in batch], end=ends)
        live = [r for r in batch if r not in ends]
        while live:
            entries = [(r, [requests[r][done[r]]], [0]) for r in live]
            for r in live:
                done[r] += 1
            ends = [r for r in live if done[r] == len(requests[r])]
            tr.add(entries, end=ends)
            live = [r for r in live if r not in ends]
    return tr


def run_trace(model_dir: Path, dtype: str, trace: Trace, out_dir: Path, max_tokens: int | None = None,
              env: dict | None = None, timeout: float = 600.0) -> dict[tuple[str, int], np.ndarray]:
    """Run bin/trace_run on the trace; returns {(request, position): logits}."""
    out_dir.mkdir(parents=True, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    run_env = dict(os.environ)
    run_env["LQ_PYTHON"] = sys.executable
    if env:
        run_env.update(env)
    proc = subprocess.run([str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(max_tokens or trace.max_tokens)],
                          input=text, capture_output=True, text=True, timeout=timeout, env=run_env)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stderr[-4000:]}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace.steps], proc.stdout[-2000:]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    result = {}
    for step, rows in trace.rows.items():
        data = np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab)
        for row, key in zip(data, rows):
            assert key not in result, f"{key} asked twice"
            result[key] = row
    for s in trace.steps:
        if s["step"] not in trace.rows:
            assert not (out_dir / f"{s['step']}.f32").exists()
    return result
