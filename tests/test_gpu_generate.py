"""Generation through the Python entry point, sampling on the device, long decoding."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY, TOL, make_model_folder, plain_logits, random_tokens, rel_err, tolerance

pytestmark = pytest.mark.gpu


def _engine(folder, dtype, **kw):
    from longbow_quarrel_b200.engine import Engine
    return Engine.from_pretrained(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw)


def _check_greedy(cfg, weights, prompt, generated, dtype, stop=()):
    """Every generated token is the plain implementation's choice (in bfloat16: a token
    whose plain logit is within the precision's tolerance of the maximum)."""
    seq = list(prompt)
    for tok in generated:
        logits = plain_llama.forward(cfg, weights, seq)[-1].numpy()
        best = int(np.argmax(logits))
        if tok != best:
            gap = (logits[best] - logits[tok]) / np.sqrt((logits ** 2).mean())
            assert dtype == "bfloat16" and gap < TOL[dtype], (len(seq), tok, best, gap)
        assert tok not in stop
        seq.append(tok)
    return seq


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_model_folder(tmp_path, name, seed=21)
    cfg, weights = plain_llama.load_folder(folder)
    eng = _engine(folder, dtype)
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 40 + i) for i, n in enumerate([7, 3, 12, 1, 20])]
    seen = []
    out = eng.generate(prompts, max_new_tokens=12, sampling=SamplingParams(temperature=0.0), stop_ids=[],
                       callback=lambda i, t: seen.append((i, t)), batch_size=3)     # two batches: slots are reused
    assert [len(o) for o in out] == [12] * 5
    for p, o in zip(prompts, out):
        _check_greedy(cfg, weights, p, o, dtype)
    assert sorted(seen) == sorted((i, t) for i, o in enumerate(out) for t in o)
    assert eng.cache.pages_in_use() == 0 and eng.cache.slots.n_live == 0
    assert eng.last_stats.batches == 2 and eng.last_stats.prompt_tokens == 43


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_token_prompts_in_reused_slots_do_not_take_the_step_queued_for_the_batch_before(tmp_path, dtype):
    """Batches of one sequence, prompts of one token: every batch gets the slot of the one before it, whose
    last step was still queued ahead.  The new prompt must run; the old request's queued token is not its first."""
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_model_folder(tmp_path, "A", seed=24)
    cfg, weights = plain_llama.load_folder(folder)
    eng = _engine(folder, dtype)
    prompts = [[5], [6], [5], [200], [17, 3], [9]]
    for batch_size in (1, 2):
        out = eng.generate(prompts, max_new_tokens=5, sampling=SamplingParams(temperature=0.0), stop_ids=[],
                           batch_size=batch_size)
        assert out[0] == out[2]
        for p, o in zip(prompts, out):
            assert len(o) == 5
            _check_greedy(cfg, weights, p, o, dtype)
    assert eng.cache.pages_in_use() == 0 and eng.cache.slots.n_live == 0


def test_logits_callback_gives_the_logits_each_token_was_chosen_from(tmp_path):
    """The counterpart of the reference's InferWithCallbackLogits: per token the logits it was sampled from, the
    plain implementation's for that position; greedy tokens are their maxima; asking for them changes no token."""
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_model_folder(tmp_path, "B", seed=27)
    eng = _engine(folder, "float32")
    prompts = [random_tokens(n, 384, 90 + i) for i, n in enumerate([6, 1, 11])]
    seen, order = {}, []

    def on_logits(i, step, logits):
        assert logits.device.type == "cpu" and logits.dtype == torch.float32 and logits.shape == (384,)
        seen[(i, step)] = logits.numpy().copy()
        order.append(("logits", i, step))
    out = eng.generate(prompts, 5, SamplingParams(), stop_ids=[], logits_callback=on_logits, batch_size=2,
                       callback=lambda i, t: order.append(("token", i, t)))
    assert out == eng.generate(prompts, 5, SamplingParams(), stop_ids=[], batch_size=2)
    assert sorted(seen) == sorted((i, s) for i in range(3) for s in range(5))
    for i, (p, o) in enumerate(zip(prompts, out)):
        ref = plain_logits(folder, p + o)
        for s, tok in enumerate(o):
            assert rel_err(seen[(i, s)], ref[len(p) + s - 1]) < TOL["float32"]
            assert int(np.argmax(seen[(i, s)])) == tok
    assert order.index(("logits", 0, 0)) < order.index(("token", 0, out[0][0]))


def test_stop_tokens_end_sequences_early(tmp_path):
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_model_folder(tmp_path, "A", seed=22)
    cfg, weights = plain_llama.load_folder(folder)
    eng = _engine(folder, "float32")
    prompts = [random_tokens(n, 256, 60 + i) for i, n in enumerate([5, 9, 2, 14])]
    free = eng.generate(prompts, 10, SamplingParams(), stop_ids=[])
    # Stop at the token that the second prompt emits third: that sequence ends after two tokens.
    stop = free[1][2]
    out = eng.generate(prompts, 10, SamplingParams(), stop_ids=[stop])
    for f, o in zip(free, out):
        cut = f.index(stop) if stop in f else len(f)
        assert o == f[:cut]
    assert out[1] == free[1][:free[1].index(stop)]
    assert eng.last_stats.finish_reasons[1] == "stop"
    # The model's own eos ids are the default.
    assert eng.model.spec.stop_tokens == (255,)


def test_long_decoding_and_first_tokens(tmp_path):
    """One prompt token, then hundreds of single-token steps: the first tokens of a
    sequence and a long run of decoding, every step's logits against plain."""
    folder = make_model_folder(tmp_path, "C", seed=23)
    tokens = random_tokens(330, 250, 5)
    ref = plain_logits(folder, tokens)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype)
        slot = eng.new_sequence()
        for i, t in enumerate(tokens):
            got = eng.step([(slot, [t])])[0].cpu().numpy()
            assert rel_err(got, ref[i]) < tolerance(dtype, folder, tokens), (dtype, i)
        eng.end_sequence(slot)


def _draws(n_rows):
    return (torch.arange(n_rows, dtype=torch.int32, device="cuda"), torch.full((n_rows,), 3, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("V", [250, 1000, 128256])
def test_sampler_matches_the_reference_rules(V):
    from longbow_quarrel_b200.sampling import SamplingParams, sample
    rng = np.random.default_rng(V)
    rows = 6
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    logits[1, 7] = logits[1].max()          # a tie for the maximum: the first wins
    dev = torch.from_numpy(logits).cuda()
    seq, step = _draws(rows)
    # greedy
    out = sample(dev, SamplingParams(temperature=0.0), seed=1).cpu().numpy()
    assert list(out) == [int(np.argmax(l)) for l in logits]
    # temperature, with and without filters
    for params in (SamplingParams(temperature=0.8, seed=11), SamplingParams(temperature=1.3, top_k=40, seed=12),
                   SamplingParams(temperature=0.7, top_p=0.9, seed=13),
                   SamplingParams(temperature=1.0, top_k=50, top_p=0.5, seed=14)):
        out = sample(dev, params, seed=params.seed, sequence_ids=seq, steps=step).cpu().numpy()
        for r in range(rows):
            u = plain_llama.philox_uniform(params.seed, r, 3)
            want = plain_llama.sample_reference(logits[r], params.temperature, params.top_k, params.top_p, u)
            if out[r] != want:
                # float32 weights against float64: the draw may fall on the other side of a boundary
                ids, probs = plain_llama.kept_set(logits[r], params.temperature, params.top_k, params.top_p)
                assert out[r] in ids, (params, r)
                c = np.cumsum(probs) / sum(probs)
                assert np.abs(c - u).min() < 1e-5, (params, r, out[r], want)


def test_sampler_top_k_one_is_greedy_and_filters_hold():
    from longbow_quarrel_b200.sampling import SamplingParams, sample
    rng = np.random.default_rng(5)
    V = 500
    logits = rng.standard_normal((1, V)).astype(np.float32)
    dev = torch.from_numpy(np.repeat(logits, 200, axis=0)).contiguous().cuda()
    seq = torch.arange(200, dtype=torch.int32, device="cuda")
    step = torch.zeros(200, dtype=torch.int32, device="cuda")
    out = sample(dev, SamplingParams(temperature=1.0, top_k=1, seed=3), 3, seq, step).cpu().numpy()
    assert set(out) == {int(np.argmax(logits[0]))}          # top-k = 1 is greedy (sampler_test.go)
    out = sample(dev, SamplingParams(temperature=1.5, top_k=5, seed=3), 3, seq, step).cpu().numpy()
    top5 = set(np.argsort(-logits[0])[:5].tolist())
    assert set(out) <= top5 and len(set(out)) > 1
    ids, _ = plain_llama.kept_set(logits[0], 1.0, 0, 0.3)
    out = sample(dev, SamplingParams(temperature=1.0, top_p=0.3, seed=3), 3, seq, step).cpu().numpy()
    assert set(out) <= set(ids)
    # the draws follow the distribution: chi-square on a small vocabulary
    small = np.log(np.array([[0.5, 0.25, 0.125, 0.125]], dtype=np.float32))
    n = 4000
    dev = torch.from_numpy(np.repeat(small, n, axis=0)).contiguous().cuda()
    out = sample(dev, SamplingParams(temperature=1.0, seed=9), 9, torch.arange(n, dtype=torch.int32, device="cuda"),
                 torch.zeros(n, dtype=torch.int32, device="cuda")).cpu().numpy()
    counts = np.bincount(out, minlength=4)
    expect = n * np.array([0.5, 0.25, 0.125, 0.125])
    assert ((counts - expect) ** 2 / expect).sum() < 16.3      # chi-square, 3 degrees of freedom, p = 0.001


@pytest.mark.parametrize("V", [2048, 5001, 128256, 300000, 500000])
def test_the_cluster_sampler_and_the_one_block_sampler_choose_the_same_tokens(V):
    """A row spread over the shared memory of a cluster of eight blocks, or in one block's scratch row in global
    memory (500,000 logits fit no cluster and take that kernel by themselves): the same rules, the same draws."""
    from longbow_quarrel_b200.sampling import SamplingParams, history_window, sample
    from longbow_quarrel_b200.sampling.sampler import needs_scratch
    assert needs_scratch(V) == (V == 500000)
    rng = np.random.default_rng(V)
    rows = 5
    logits = (rng.standard_normal((rows, V)) * 4).astype(np.float32)
    logits[0, V - 1] = logits[0].max() + 1.0        # the maximum in the last block's part
    logits[2, 700:720] = logits[2].max()            # twenty equal weights at the top: ties at a top-k cut-off
    dev = torch.from_numpy(logits).cuda()
    seq = torch.arange(rows, dtype=torch.int32, device="cuda")
    step = torch.full((rows,), 7, dtype=torch.int32, device="cuda")
    hist, n = history_window([list(range(i, i + 40)) + [V - 1] for i in range(rows)])
    hist, n = torch.from_numpy(hist).cuda(), torch.from_numpy(n).cuda()
    for params in (SamplingParams(), SamplingParams(temperature=1.0, seed=4), SamplingParams(temperature=0.6, top_k=40, seed=5),
                   SamplingParams(temperature=0.6, top_k=7, seed=5), SamplingParams(temperature=1.2, top_p=0.9, seed=6),
                   SamplingParams(temperature=0.7, top_k=40, top_p=0.95, repetition_penalty=1.3, seed=7),
                   SamplingParams(repetition_penalty=5.0)):
        kw = dict(history=hist, history_len=n) if params.uses_history else {}
        for offset in (0, 3):
            a = sample(dev, params, params.seed or 1, seq, step, step_offset=offset, **kw).cpu().numpy()
            b = sample(dev, params, params.seed or 1, seq, step, step_offset=offset, one_block=True, **kw).cpu().numpy()
            assert list(a) == list(b), (params, offset)
    bad = logits.copy()
    bad[1, :V // 2] = np.nan
    bad[3, 5] = np.inf
    for one_block in (False, True):
        out = sample(torch.from_numpy(bad).cuda(), SamplingParams(temperature=0.9, seed=2), 2, seq, step, one_block=one_block)
        assert list(out.cpu().numpy()[[1, 3]]) == [V // 2, 0]


def test_sampler_penalty_and_bad_logits():
    from longbow_quarrel_b200.sampling import SamplingParams, history_window, sample
    logits = np.array([[1.0, 3.0, 2.9, -1.0], [1.0, -0.5, -0.6, -2.0]], dtype=np.float32)
    hist, n = history_window([[1, 1, 0], [1]])
    dev = torch.from_numpy(logits).cuda()
    out = sample(dev, SamplingParams(temperature=0.0, repetition_penalty=2.0), 1, history=torch.from_numpy(hist).cuda(),
                 history_len=torch.from_numpy(n).cuda()).cpu().numpy()
    ref = [int(np.argmax(plain_llama.repetition_penalty(logits[0], [1, 1, 0], 2.0))),
           int(np.argmax(plain_llama.repetition_penalty(logits[1], [1], 2.0)))]
    assert list(out) == ref == [2, 0]
    bad = np.array([[np.nan, np.inf, 0.5, 9.0], [1.0, 2.0, np.nan, 0.0]], dtype=np.float32)
    out = sample(torch.from_numpy(bad).cuda(), SamplingParams(temperature=0.0), 1).cpu().numpy()
    assert list(out) == [2, 0]            # the first finite index (internal/engine/sampler.go:116-123)


def test_temperature_generation_is_reproducible_and_independent_of_the_batch(tmp_path):
    from longbow_quarrel_b200.sampling import SamplingParams
    folder = make_model_folder(tmp_path, "B", seed=24)
    eng = _engine(folder, "float32")
    prompts = [random_tokens(n, 384, 80 + i) for i, n in enumerate([20, 5, 33])]
    params = SamplingParams(temperature=0.8, seed=1234)
    a = eng.generate(prompts, 16, params, stop_ids=[])
    b = eng.generate(prompts, 16, params, stop_ids=[])
    assert a == b                                             # same seed, same tokens
    c = eng.generate(prompts, 16, SamplingParams(temperature=0.8, seed=99), stop_ids=[])
    assert a != c
    alone = eng.generate(prompts, 16, params, stop_ids=[], batch_size=1)
    # request i draws from its own stream whatever the batch; in 32-bit the logits agree to
    # rounding, so the sampled tokens agree
    assert alone == a
    # every sampled token is one the plain implementation's distribution allows
    cfg, weights = plain_llama.load_folder(folder)
    for i, (p, o) in enumerate(zip(prompts, a)):
        seq = list(p)
        for step, tok in enumerate(o):
            logits = plain_llama.forward(cfg, weights, seq)[-1].numpy()
            u = plain_llama.philox_uniform(1234, i, step)
            want = plain_llama.sample_reference(logits, 0.8, 0, 1.0, u)
            if tok != want:
                ids, probs = plain_llama.kept_set(logits, 0.8, 0, 1.0)
                c = np.cumsum(probs)
                assert np.abs(c - u).min() < 1e-4, (i, step)
            seq.append(tok)


def test_smoke_entry_point():
    import __graft_entry__
    __graft_entry__.smoke()


def test_command_line_generates_the_plain_implementations_tokens(tmp_path):
    """bin/quarrel with the reference's option names, greedy, two prompts, JSON output."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    folder = make_model_folder(tmp_path, "A", seed=25)
    cfg, weights = plain_llama.load_folder(folder)
    exe = Path(__file__).resolve().parent.parent / "bin" / "quarrel"
    proc = subprocess.run([str(exe), "-model", str(folder), "-prompt-ids", "3,1,4,1,5;9,2,6", "-n", "6", "-temp", "0",
                           "-dtype", "float32", "-output", "json", "-kv-cache-size", "64"],
                          capture_output=True, text=True, timeout=300, env={**os.environ, "LQ_PYTHON": sys.executable})
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["tokens_generated"] == 12 and set(out) >= {"throughput_tokens_per_sec", "prefill_duration_seconds",
                                                          "generation_duration_seconds", "total_duration_seconds"}
    for prompt, new in zip(([3, 1, 4, 1, 5], [9, 2, 6]), out["output"]):
        assert new == plain_llama.greedy(cfg, weights, prompt, 6)       # config A names no bos token: none is added
    text = subprocess.run([str(exe), "-model", str(folder), "-prompt", "Hi", "-n", "3", "-temp", "0.7", "-topk", "40",
                           "-topp", "0.95", "-penalty", "1.1", "-seed", "7", "-stream"], capture_output=True, text=True,
                          timeout=300, env={**os.environ, "LQ_PYTHON": sys.executable})
    assert text.returncode == 0 and "3 tokens in" in text.stdout and "Longbow-Quarrel" in text.stdout


def test_bench_command_with_a_prompt_file(tmp_path):
    """`quarrel bench`: greedy, the reference's JSON fields, prompts from a file; and the timeout."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    folder = make_model_folder(tmp_path, "A", seed=26)
    cfg, weights = plain_llama.load_folder(folder)
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("3 1 4 1 5\n9,2,6\n")
    exe = Path(__file__).resolve().parent.parent / "bin" / "quarrel"
    env = {**os.environ, "LQ_PYTHON": sys.executable}
    proc = subprocess.run([str(exe), "bench", "-model", str(folder), "-prompt-file", str(prompts), "-tokens", "5",
                           "-dtype", "float32", "-output", "json"], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["tokens_generated"] == 10 and out["throughput_tokens_per_sec"] > 0
    assert out["prefill_duration_seconds"] + out["generation_duration_seconds"] == pytest.approx(out["total_duration_seconds"])
    for prompt, new in zip(([3, 1, 4, 1, 5], [9, 2, 6]), out["output"]):
        assert new == plain_llama.greedy(cfg, weights, prompt, 5)
    late = subprocess.run([str(exe), "bench", "-model", str(folder), "-prompt-len", "8", "-batch", "2", "-tokens", "50",
                           "-timeout", "0"], capture_output=True, text=True, timeout=300, env=env)
    assert late.returncode == 1 and "timed out after 0 seconds" in late.stderr
