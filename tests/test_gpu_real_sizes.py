"""Layers of the sizes that real checkpoints have, through bin/trace_run against the plain
implementation: two layers of the Llama-3.1-8B shape (hidden 4096, 32 heads over 8 kv heads of 128,
intermediate 14336) and of the Llama-3.2-1B shape (hidden 2048, heads of 64, tied head), the vocabulary
cut to a few thousand so that the float64 plain model runs on the CPU.  These sizes take the kernels
that the tiny configurations never reach -- the tcgen05 products with rotation and cache write in their
epilogue, the tcgen05 prompt attention, the streamed products of decode steps with folded norms -- and the
test asserts from the replay program's kernel counts that they ran.

Every request is replayed whole, with its last tokens one by one, in batches of unequal prompts whose
members end at different steps and whose slots a second batch takes over, and with its prompt cut into
several steps; all cuts run in ONE call of the replay program, so a slot or page that one cut leaves
is what the next one gets.  Stored expectations per position are the plain implementation's logits, made
when the test runs (the reference's regression files, cmd/smoke_test/regression_suite.go:22-64, are the
seed: prompt -> expected logits, compared by their difference).
"""
import numpy as np
import pytest

import plain_llama
from helpers import REAL, Errors, bounds, make_model_folder, random_tokens, rel_err, rel_l2, storage_noise
from trace_tools import (Trace, kernel_class, kernel_counts, layer_stats, run_trace, split, trace_batches, trace_chunked,
                         trace_last_one_by_one, trace_whole)

pytestmark = pytest.mark.gpu

# prompt length, decoded tokens: a prompt of one token, prompts around the page size of 64 and the query
# tiles of 64 and 128, a long one of an odd length, and the benchmark's 2,048
REQUESTS = {"p1": (1, 32), "p17": (17, 20), "p64": (64, 32), "p65": (65, 8), "p700": (700, 32), "p2048": (2048, 32)}
SECOND_BATCH = {"q300": (300, 8), "q3": (3, 8), "q129": (129, 4)}


def _wanted(n):
    """Of n tokens fed in one step: the first three, every 61st, and the last 33 (a prompt's end and what follows)."""
    return sorted(set(range(min(3, n))) | set(range(0, n, 61)) | set(range(max(0, n - 33), n)))


_made = {}


def _model(tmp_path_factory, shape):
    """Model folder, requests and the plain implementation's logits, made once per shape."""
    if shape not in _made:
        folder = make_model_folder(tmp_path_factory.mktemp(f"real_{shape}"), shape, seed=31)
        vocab = REAL[shape]["vocab_size"]
        requests = {rid: random_tokens(p + d, vocab, 500 + i)
                    for i, (rid, (p, d)) in enumerate({**REQUESTS, **SECOND_BATCH}.items())}
        cfg, weights = plain_llama.load_folder(folder)
        weights = {name: t.double() for name, t in weights.items()}        # once, not once per request
        ref, hidden = {}, {}
        for rid, tokens in requests.items():
            ref[rid], hidden[rid] = plain_llama.forward(cfg, weights, tokens, return_layers=True)
        # the yardstick for bfloat16: the storage noise of three requests of different lengths
        noise = [storage_noise(cfg, weights, requests[r], ref[r]) for r in ("p64", "q300", "p700")]
        _made[shape] = (folder, requests, ref, hidden, (max(n[0] for n in noise), max(n[1] for n in noise)), (cfg, weights))
    return _made[shape]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["1B", "8B"])
def test_real_layer_sizes_in_every_cut(tmp_path_factory, tmp_path, shape, dtype):
    folder, requests, ref, hidden, noise, _ = _model(tmp_path_factory, shape)
    first = {r: requests[r] for r in REQUESTS}
    prompt = {r: p for r, (p, _) in {**REQUESTS, **SECOND_BATCH}.items()}

    tr = Trace()
    tr.extend(trace_whole(first, _wanted), "whole:")
    tail = Trace()
    for rid, tokens in first.items():
        p = prompt[rid]
        tail.add([(rid, tokens[:p], [p - 1])])
        for i in range(p, len(tokens)):
            tail.add([(rid, [tokens[i]], [0])], end=[rid] if i == len(tokens) - 1 else [])
    tr.extend(tail, "tail:")
    tr.extend(trace_batches(requests, prompt, width=6, want=_wanted), "batch:")      # six, then three in their slots
    tr.extend(trace_chunked({r: requests[r] for r in ("p700", "q300")}, [130, 2, 17, 200], n_single=4), "chunk:")
    out = tmp_path / "out"
    got = run_trace(folder, dtype, tr, out, options=["--kernel-counts", "--layer-stats"], timeout=900)

    errs = Errors()
    whole, tail, batch = split(got, "whole:"), split(got, "tail:"), split(got, "batch:")
    for cut in ("whole:", "tail:", "batch:", "chunk:"):
        rows = split(got, cut)
        assert rows, cut
        for (rid, pos), row in rows.items():
            errs.add(f"plain max {cut}", rel_err(row, ref[rid][pos]), (rid, pos))
            errs.add(f"plain l2 {cut}", rel_l2(row, ref[rid][pos]), (rid, pos))
    # The cuts against one another, position by position: "same" where both results come from the same
    # family of kernels (another batch around them, another cut of the prompt), "other" where they do not
    # (a position once as part of a prompt, once decoded; a step of few rows and one of many).
    shapes = {cut: split(tr.shape, cut) for cut in ("whole:", "tail:", "batch:", "chunk:")}
    cuts = {"whole:": whole, "tail:": tail, "batch:": batch, "chunk:": split(got, "chunk:")}
    for a, b_ in (("tail:", "whole:"), ("batch:", "whole:"), ("batch:", "tail:"), ("chunk:", "whole:"), ("chunk:", "batch:")):
        for key, row in cuts[a].items():
            if key in cuts[b_]:
                same = kernel_class(*shapes[a][key]) == kernel_class(*shapes[b_][key])
                kind = "same" if same else "other"
                errs.add(f"{kind} max {a}{b_}", rel_err(row, cuts[b_][key]), key)
                errs.add(f"{kind} l2 {a}{b_}", rel_l2(row, cuts[b_][key]), key)
    print(f"\n[{shape} {dtype}] storage noise l2 {noise[0]:.3g} max {noise[1]:.3g}; {errs}")
    errs.check(bounds(dtype, noise))

    # the residual stream after every layer, where a wrong layer would show first
    stats = layer_stats(out, tr)
    for (rid, pos), rms in split(stats, "tail:").items():
        want = np.sqrt((hidden[rid][:, pos] ** 2).mean(axis=1))
        assert rms.shape == want.shape == (REAL[shape]["num_hidden_layers"] + 1,)
        assert np.abs(rms - want).max() < (1e-4 if dtype == "float32" else 1.5 * noise[0]) * want.max(), (rid, pos, rms, want)

    counts = kernel_counts(out)
    if dtype == "bfloat16":
        for name in ("gemm_tc_qkv", "gemm_pair_qkv", "gemm_pair", "attn_prefill_tc", "gemm_skinny_qkv", "attn_decode", "gemm_tc", "gemm_skinny",
                     "gemm_skinny:rows8:norm_in", "attn_decode:teams"):
            assert counts.get(name, 0) > 0, (name, counts)
        assert "attention" not in counts and "linear" not in counts, counts       # no plain kernel took a product
    else:
        assert not any(k.startswith(("gemm_tc", "gemm_skinny", "attn_")) for k in counts), counts


POOL_WIDTHS = (12, 17, 33, 64, 100)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_batches_at_real_layer_sizes(tmp_path_factory, tmp_path, dtype):
    """133 short requests at the 1B shape, run in batches of 12, 17, 33, 64 and 100 that start together with
    unequal prompts; members end at different steps and every later batch starts in slots that were given
    back.  Each width takes other kernels for its decode steps: 9 to 16 rows stream the weights through
    registers in two row tiles, 17 rows and more take the tcgen05 kernel (the contraction cut into ranges
    where the weight is narrow), and from 19 sequences on the decode attention runs one slice per sequence.
    Every (request, position) must agree with the plain implementation and, across widths, with itself."""
    folder, _, _, _, _, (cfg, weights) = _model(tmp_path_factory, "1B")
    vocab = REAL["1B"]["vocab_size"]
    rng = np.random.default_rng(77)
    lengths = [int(n) for n in rng.integers(2, 30, 133)]
    lengths[5], lengths[40] = 140, 70                         # two that cross pages
    pool = {f"s{i}": random_tokens(n, vocab, 900 + i) for i, n in enumerate(lengths)}
    prompt = {r: int(rng.integers(1, min(len(t), 24) + 1)) for r, t in pool.items()}
    prompt["s5"] = 130
    ref = {r: plain_llama.forward(cfg, weights, t).numpy() for r, t in pool.items()}
    noise = [storage_noise(cfg, weights, pool[r], ref[r]) for r in ("s5", "s40", "s0", "s1", "s2", "s3")]
    noise = (max(n[0] for n in noise), max(n[1] for n in noise))

    tr = Trace()
    for w in POOL_WIDTHS:
        tr.extend(trace_batches(pool, prompt, width=w), f"w{w}:")
    out = tmp_path / "out"
    got = run_trace(folder, dtype, tr, out, options=["--kernel-counts"], timeout=900)
    assert len(got) == len(POOL_WIDTHS) * sum(lengths)
    base = split(got, f"w{POOL_WIDTHS[0]}:")
    errs = Errors()
    for w in POOL_WIDTHS:
        for (rid, pos), row in split(got, f"w{w}:").items():
            errs.add(f"plain max w{w}", rel_err(row, ref[rid][pos]), (rid, pos))
            errs.add(f"plain l2 w{w}", rel_l2(row, ref[rid][pos]), (rid, pos))
            same = kernel_class(*tr.shape[(f"w{w}:{rid}", pos)]) == kernel_class(*tr.shape[(f"w{POOL_WIDTHS[0]}:{rid}", pos)])
            kind = "same" if same else "other"
            errs.add(f"{kind} max w{w}:w{POOL_WIDTHS[0]}", rel_err(row, base[(rid, pos)]), (rid, pos))
            errs.add(f"{kind} l2 w{w}:w{POOL_WIDTHS[0]}", rel_l2(row, base[(rid, pos)]), (rid, pos))
    print(f"\n[1B {dtype} widths] storage noise l2 {noise[0]:.3g} max {noise[1]:.3g}; {errs}")
    errs.check(bounds(dtype, noise))
    if dtype == "bfloat16":
        counts = kernel_counts(out)
        for name in ("gemm_skinny:rows16", "gemm_skinny_qkv:rows16", "gemm_tc:split_k", "gemm_tc_qkv:split_k",
                     "attn_decode:teams", "attn_prefill_tc"):
            assert counts.get(name, 0) > 0, (name, counts)
