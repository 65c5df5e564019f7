"""Trace replay through bin/trace_run: the same requests whole, with the last 32
tokens one by one, and in batches of unequal lengths whose slots are used again,
in 32-bit and in bfloat16, all against the plain implementation."""
import pytest

from helpers import TINY, TOL, make_model_folder, plain_logits, random_tokens, rel_err, tolerance
from trace_tools import Trace, run_trace, split, trace_batches, trace_last_one_by_one, trace_whole

pytestmark = pytest.mark.gpu

# Two cuts in bfloat16 come from other kernels, which sum in another order; a difference far below a rounding
# step becomes a whole step where it tips a rounding, so after a few operations two correct paths are as far
# apart as rounding noise itself (tests/helpers.py: storage_noise).  In float32 the cuts are equal bit by bit.

LENGTHS = {"r0": 40, "r1": 33, "r2": 100, "r3": 57, "r4": 71, "r5": 34, "r6": 90}
PROMPTS = {"r0": 7, "r1": 33, "r2": 12, "r3": 1, "r4": 64, "r5": 20, "r6": 65}


def _requests(name):
    vocab = TINY[name]["vocab_size"]
    return {rid: random_tokens(n, vocab, 100 + i) for i, (rid, n) in enumerate(LENGTHS.items())}


def _compare(got, requests, folder, dtype, what):
    worst = 0.0
    for rid, tokens in requests.items():
        ref = plain_logits(folder, tokens)
        tol = tolerance(dtype, folder, tokens)
        for pos in range(len(tokens)):
            if (rid, pos) in got:
                err = rel_err(got[(rid, pos)], ref[pos])
                worst = max(worst, err)
                assert err < tol, f"{what}: request {rid} position {pos} of {len(tokens)}: error {err:.3g}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_all_cuts_match_plain(tmp_path, name, dtype):
    folder = make_model_folder(tmp_path, name, seed=11)
    requests = _requests(name)
    # One call of the replay program serves the three cuts, one after the other: each starts in the slots
    # and pages that the one before it gave back.
    tr = Trace()
    tr.extend(trace_whole(requests), "whole:")
    tr.extend(trace_last_one_by_one(requests), "tail:")
    tr.extend(trace_batches(requests, PROMPTS, width=3), "batched:")
    got = run_trace(folder, dtype, tr, tmp_path / "out")
    whole, tail, batched = split(got, "whole:"), split(got, "tail:"), split(got, "batched:")
    assert len(whole) == sum(LENGTHS.values())
    _compare(whole, requests, folder, dtype, "whole")
    assert len(tail) == 33 * len(requests)
    _compare(tail, requests, folder, dtype, "last 32 one by one")
    assert len(batched) == sum(LENGTHS.values())
    _compare(batched, requests, folder, dtype, "unequal batches")

    # The cuts against one another: equal in float32 (to 2e-5; in practice bit by bit), within the same noise in bfloat16.
    for key, row in tail.items():
        cut_tol = 2e-5 if dtype == "float32" else tolerance(dtype, folder, requests[key[0]])
        assert rel_err(row, whole[key]) < cut_tol, ("tail vs whole", key)
    for key, row in batched.items():
        cut_tol = 2e-5 if dtype == "float32" else tolerance(dtype, folder, requests[key[0]])
        assert rel_err(row, whole[key]) < cut_tol, ("batched vs whole", key)


def test_max_tokens_sizes_the_cache_exactly(tmp_path):
    """--max-tokens is the most tokens live requests hold, each rounded up to 64: the trace runs
    with exactly that, and is refused with one page less."""
    import subprocess
    import sys

    from trace_tools import TRACE_RUN, Trace
    folder = make_model_folder(tmp_path, "A", seed=12)
    tr = Trace()
    a, b, c = random_tokens(70, 256, 1), random_tokens(64, 256, 2), random_tokens(10, 256, 3)
    tr.add([("a", a, [69]), ("b", b, [63])])                  # 128 + 64 tokens held
    tr.add([("a", [5], [0]), ("b", [6], [0])], end=["a"])     # b grows into a second page: 128 + 128
    tr.add([("b", [7], [0]), ] , end=[])                      # a's pages are back: 128 held
    tr.add([("c", c, [9])], end=["b", "c"])                   # a new request takes freed pages: 128 + 64
    assert tr.max_tokens == 256
    got = run_trace(folder, "float32", tr, tmp_path / "exact", max_tokens=256)
    ref = plain_logits(folder, a + [5])
    assert rel_err(got[("a", 70)], ref[70]) < TOL["float32"]
    ref = plain_logits(folder, c)
    assert rel_err(got[("c", 9)], ref[9]) < TOL["float32"]
    import json
    text = "".join(json.dumps(s) + "\n" for s in tr.steps)
    proc = subprocess.run([str(TRACE_RUN), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "small"),
                           "--max-tokens", "192"], input=text, capture_output=True, text=True, timeout=300,
                          env={**__import__("os").environ, "LQ_PYTHON": sys.executable})
    assert proc.returncode != 0 and "cache is full" in proc.stderr
    assert proc.stdout.splitlines() == ["done 0"]             # the first step fits; the second does not
