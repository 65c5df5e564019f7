"""Ways of cutting and batching that generation itself never produces but the step function accepts, on
tiny configurations that take the kernels of real models (head sizes 64 and 128): prompts fed in several
steps, steps that mix a continuation of several tokens with single tokens, wide batches whose members end
at different steps, pages that come back holding another request's values, and a long run of
graph-replayed single-token steps on a model of one layer."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import (TINY, TOL, Errors, assert_rows_close, bounds, tolerance, make_model_folder, plain_logits, random_tokens, rel_err, rel_l2,
                     storage_noise)
from trace_tools import Trace, kernel_counts, run_trace, split, trace_batches, trace_chunked, trace_mixed, trace_whole

pytestmark = pytest.mark.gpu


def _requests(vocab, lengths, seed, name="r"):
    return {f"{name}{i}": random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_in_portions_mixed_steps_and_wide_batches(tmp_path, dtype):
    """Config D: head_dim 64, a window of 100 on every other layer.  All cuts run in one call of the replay
    program, one after the other, so each starts in the slots and pages the last one gave back."""
    folder = make_model_folder(tmp_path, "D", seed=41, std=0.1)         # large weights: one wrong key shows
    vocab = TINY["D"]["vocab_size"]
    rng = np.random.default_rng(41)
    long_ = _requests(vocab, [330, 200, 131, 64], 700)                   # past the window and several pages
    pool = _requests(vocab, [int(n) for n in rng.integers(2, 60, 45)], 800, "s")
    prompt = {r: int(rng.integers(1, len(t) + 1)) for r, t in pool.items()}
    cfg, weights = plain_llama.load_folder(folder)
    weights = {name: t.double() for name, t in weights.items()}
    ref = {r: plain_llama.forward(cfg, weights, t).numpy() for r, t in {**long_, **pool}.items()}
    noise = [storage_noise(cfg, weights, t, ref[r]) for r, t in {**long_, **pool}.items()]
    noise = (max(n[0] for n in noise), max(n[1] for n in noise))

    tr = Trace()
    tr.extend(trace_whole(long_), "whole:")
    tr.extend(trace_chunked(long_, [130, 2, 17, 90], n_single=40), "chunk:")      # 130 + 2 + 17 + 90 ..., then one by one
    tr.extend(trace_mixed(long_, {"r0": 70, "r1": 1, "r2": 128, "r3": 64}, [5, 1, 1, 33]), "mixed:")
    tr.extend(trace_batches(pool, prompt, width=9), "w9:")
    tr.extend(trace_batches(pool, prompt, width=33), "w33:")             # 33, then 12 in slots that were given back
    tr.extend(trace_whole(pool), "pool:")
    out = tmp_path / "out"
    got = run_trace(folder, dtype, tr, out, options=["--kernel-counts"])
    assert len(got) == 3 * sum(len(t) for t in long_.values()) + 3 * sum(len(t) for t in pool.values())

    errs = Errors()
    for cut in ("whole:", "chunk:", "mixed:", "w9:", "w33:", "pool:"):
        for (rid, pos), row in split(got, cut).items():
            errs.add(f"plain max {cut}", rel_err(row, ref[rid][pos]), (rid, pos))
            errs.add(f"plain l2 {cut}", rel_l2(row, ref[rid][pos]), (rid, pos))
    for cut, base in (("chunk:", "whole:"), ("mixed:", "whole:"), ("w9:", "pool:"), ("w33:", "pool:")):
        want = split(got, base)
        for key, row in split(got, cut).items():
            errs.add(f"other max {cut}{base}", rel_err(row, want[key]), key)
            errs.add(f"other l2 {cut}{base}", rel_l2(row, want[key]), key)
    print(f"\n[D {dtype}] storage noise l2 {noise[0]:.3g} max {noise[1]:.3g}; {errs}")
    errs.check(bounds(dtype, noise))
    if dtype == "bfloat16":
        counts = kernel_counts(out)
        for name in ("attn_prefill_tc", "gemm_tc_qkv", "gemm_skinny_qkv:rows16", "gemm_skinny:rows16", "gemm_tc:few_rows",
                     "gemm_tc_qkv:few_rows", "attn_decode:teams"):
            assert counts.get(name, 0) > 0, (name, counts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_that_come_back_holding_nan_do_not_reach_the_next_request(tmp_path, dtype):
    """The prompt kernel on the tensor cores loads whole pages and multiplies rows beyond a sequence's
    length by probability zero; so a page handed out again must not show what its last owner (or anyone)
    left in it.  Every free page is filled with NaN on the host's side of the test before a shorter
    request takes two of them."""
    from longbow_quarrel_b200.engine import Engine
    folder = make_model_folder(tmp_path, "D", seed=42)
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    vocab = TINY["D"]["vocab_size"]
    first, second = random_tokens(190, vocab, 1), random_tokens(70, vocab, 2)
    slot = eng.new_sequence()
    eng.step([(slot, first)])
    eng.end_sequence(slot)
    for g in eng.cache.kv_groups:                       # everything is free now: poison every page
        assert g.n_free_pages == g.n_pages
        g.k_pages.fill_(float("nan"))
        g.v_pages.fill_(float("nan"))
    ref = plain_logits(folder, second + [3, 4, 5])
    slot = eng.new_sequence()
    tol = tolerance(dtype, folder, second + [3, 4, 5])
    got = eng.step([(slot, second)], want=[list(range(70))]).cpu().numpy()      # 64 + 6 tokens: the second page's end is unwritten
    assert_rows_close(got, ref[:70], tol, "prompt in reused pages")
    for i, t in enumerate([3, 4, 5]):
        got = eng.step([(slot, [t])]).cpu().numpy()[0]
        assert rel_err(got, ref[70 + i]) < tol, i
    # a continuation of several tokens that reaches into a third, new page
    more = random_tokens(60, vocab, 3)
    ref = plain_logits(folder, second + [3, 4, 5] + more)
    got = eng.step([(slot, more)], want=[list(range(60))]).cpu().numpy()
    assert_rows_close(got, ref[73:], tolerance(dtype, folder, second + [3, 4, 5] + more), "continuation into a new page")
    eng.end_sequence(slot)
    eng.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_head_size_128_decoded_for_hundreds_of_graph_replayed_steps(tmp_path, dtype):
    """With one layer the cache write of a step is only a handful of kernels ahead of the next step's
    attention, which asks for earlier keys before it waits for the kernel ahead of it: every one of several
    hundred replayed steps must still see all of its keys.  Two sequences side by side, unequal in length."""
    from longbow_quarrel_b200.engine import Engine
    folder = make_model_folder(tmp_path, "E", seed=43, std=0.1)
    vocab = TINY["E"]["vocab_size"]
    a, b = random_tokens(420, vocab, 5), random_tokens(300, vocab, 6)
    cfg, weights = plain_llama.load_folder(folder)
    ref_a, ref_b = plain_logits(folder, a), plain_logits(folder, b)
    noise = [storage_noise(cfg, weights, t, r) for t, r in ((a, ref_a), (b, ref_b))]
    noise = (max(n[0] for n in noise), max(n[1] for n in noise))
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024)
    assert eng.stepper.use_graphs
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got = eng.step([(sa, a[:3]), (sb, b[:70])]).cpu().numpy()
    first_tol = bounds(dtype, noise)["plain max"] if dtype == "bfloat16" else TOL[dtype]
    assert rel_err(got[0], ref_a[2]) < first_tol and rel_err(got[1], ref_b[69]) < first_tol
    logits = []
    for i in range(230):                                  # queued back to back: the host reads nothing in between
        logits.append(eng.step([(sa, [a[3 + i]]), (sb, [b[70 + i]])]).clone())
    eng.end_sequence(sb)
    for i in range(230, 417):
        logits.append(eng.step([(sa, [a[3 + i]])]).clone())
    torch.cuda.synchronize()
    eng.check()
    errs = Errors()
    for i, row in enumerate(logits):
        row = row.cpu().numpy()
        errs.add("plain max a", rel_err(row[0], ref_a[3 + i]), i)
        errs.add("plain l2 a", rel_l2(row[0], ref_a[3 + i]), i)
        if i < 230:
            errs.add("plain max b", rel_err(row[1], ref_b[70 + i]), i)
            errs.add("plain l2 b", rel_l2(row[1], ref_b[70 + i]), i)
    print(f"\n[E {dtype} long decode] storage noise l2 {noise[0]:.3g} max {noise[1]:.3g}; {errs}")
    errs.check(bounds(dtype, noise))
    from longbow_quarrel_b200.kernels import ops
    assert len(eng.stepper._graphs) == 2                  # one captured step for two sequences, one for one
