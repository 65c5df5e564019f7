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
        self.shape: dict[tuple[str, int], tuple[int, int]] = {}     # (request, position) -> (rows of its step, most rows of one request)
        self._live: dict[str, int] = {}

    def add(self, entries: list[tuple[str, list[int], list[int]]], end: list[str] = ()):
        """entries: (request id, tokens, wanted places among them)."""
        step = len(self.steps)
        rows = []
        for rid, tokens, want in entries:
            start = self._live.get(rid, 0)
            self._live[rid] = start + len(tokens)
            rows += [(rid, start + w) for w in want]
        total, most = sum(len(t) for _, t, _ in entries), max((len(t) for _, t, _ in entries), default=0)
        for key in rows:
            self.shape[key] = (total, most)
        self.max_tokens = max(self.max_tokens, sum(round64(n) for n in self._live.values()))
        self.steps.append({"step": step, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries],
                           "end": list(end)})
        if rows:
            self.rows[step] = rows
        for rid in end:
            del self._live[rid]


    def extend(self, other: "Trace", prefix: str) -> None:
        """Append the steps of another trace, its request ids prefixed (so that one run of the replay
        program serves several ways of cutting the same requests).  `other` must have ended all its requests."""
        assert not self._live and not other._live
        for s in other.steps:
            step = len(self.steps)
            self.steps.append({"step": step, "entries": [{**e, "id": prefix + e["id"]} for e in s["entries"]],
                               "end": [prefix + r for r in s["end"]]})
            if s["step"] in other.rows:
                self.rows[step] = [(prefix + rid, pos) for rid, pos in other.rows[s["step"]]]
        self.shape.update({(prefix + rid, pos): v for (rid, pos), v in other.shape.items()})
        self.max_tokens = max(self.max_tokens, other.max_tokens)


def kernel_class(rows_of_step: int, most_rows_of_a_request: int) -> str:
    """Which family of bfloat16 kernels a step of this shape takes: steps of one token per request take
    the decode attention, all others the prompt attention; up to 8 rows the products stream the weights
    through registers and fold the norms, up to 16 they stream without folding, above that they run on
    tcgen05.  Two results of one position from steps of the same class come from the same kernels."""
    kind = "decode" if most_rows_of_a_request == 1 else "prompt"
    rows = "rows<=8" if rows_of_step <= 8 else "rows<=16" if rows_of_step <= 16 else "rows>16"
    return f"{kind} {rows}"


def split(result: dict, prefix: str) -> dict:
    """The rows of one of the traces that `Trace.extend` put together."""
    return {(rid[len(prefix):], pos): row for (rid, pos), row in result.items() if rid.startswith(prefix)}


def trace_whole(requests: dict[str, list[int]], want=None) -> Trace:
    """Each request alone, all of its tokens in one step, logits everywhere (or at want(n) of n tokens)."""
    tr = Trace()
    for rid, tokens in requests.items():
        tr.add([(rid, tokens, list(range(len(tokens))) if want is None else want(len(tokens)))], end=[rid])
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


def trace_chunked(requests: dict[str, list[int]], chunks: list[int], n_single: int = 0) -> Trace:
    """Each request alone, its tokens in steps of chunks[0], chunks[1], ... tokens (the last chunk size
    repeats; sizes of one are single-token steps), the last n_single tokens one a step; logits everywhere."""
    tr = Trace()
    for rid, tokens in requests.items():
        at, i, body = 0, 0, len(tokens) - n_single
        while at < len(tokens):
            n = min(chunks[min(i, len(chunks) - 1)], body - at) if at < body else 1
            tr.add([(rid, tokens[at:at + n], list(range(n)))], end=[rid] if at + n == len(tokens) else [])
            at, i = at + n, i + 1
    return tr


def trace_mixed(requests: dict[str, list[int]], prompt_len: dict[str, int], portions: list[int]) -> Trace:
    """All requests start together with unequal prompts; afterwards request k brings portions[(k + step) %
    len(portions)] tokens a step (several tokens beside single tokens in one step) until it runs out; a
    request that is finished ends, the others go on.  Logits everywhere."""
    tr = Trace()
    ids = list(requests)
    done = {r: prompt_len[r] for r in ids}
    ends = [r for r in ids if done[r] == len(requests[r])]
    tr.add([(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in ids], end=ends)
    live, step = [r for r in ids if r not in ends], 0
    while live:
        entries = []
        for k, r in enumerate(live):
            n = min(portions[(k + step) % len(portions)], len(requests[r]) - done[r])
            entries.append((r, requests[r][done[r]:done[r] + n], list(range(n))))
            done[r] += n
        ends = [r for r in live if done[r] == len(requests[r])]
        tr.add(entries, end=ends)
        live, step = [r for r in live if r not in ends], step + 1
    return tr


def trace_batches(requests: dict[str, list[int]], prompt_len: dict[str, int], width: int, want=None) -> Trace:
    """Batches of `width` requests that start together with unequal prompts, then go on
    one token each; a request that runs out of tokens ends, the others go on; when a
    batch is over the next one starts (in the slots that were given back)."""
    tr = Trace()
    ids = list(requests)
    for b0 in range(0, len(ids), width):
        batch = ids[b0:b0 + width]
        done = {r: prompt_len[r] for r in batch}
        ends = [r for r in batch if done[r] == len(requests[r])]
        tr.add([(r, requests[r][:prompt_len[r]], list(range(prompt_len[r])) if want is None else want(prompt_len[r]))
                for r in batch], end=ends)
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
              env: dict | None = None, timeout: float = 600.0, options: list[str] = ()) -> dict[tuple[str, int], np.ndarray]:
    """Run bin/trace_run on the trace; returns {(request, position): logits}.  `options`: further
    arguments (--layer-stats, --kernel-counts; what they write is read with `layer_stats`, `kernel_counts`)."""
    out_dir.mkdir(parents=True, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    run_env = dict(os.environ)
    run_env["LQ_PYTHON"] = sys.executable
    if env:
        run_env.update(env)
    proc = subprocess.run([str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(max_tokens or trace.max_tokens), *options],
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


def layer_stats(out_dir: Path, trace: Trace) -> dict[tuple[str, int], np.ndarray]:
    """{(request, position): RMS of the residual stream after the embedding and after every layer}."""
    result = {}
    for step, rows in trace.rows.items():
        data = np.fromfile(out_dir / f"{step}.layers.f32", dtype="<f4").reshape(len(rows), -1)
        for row, key in zip(data, rows):
            result[key] = row
    return result


def kernel_counts(out_dir: Path) -> dict[str, int]:
    return json.loads((out_dir / "kernels.json").read_text())
