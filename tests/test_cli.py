"""The command line's options: the reference's names, defaults and meanings
(cmd/quarrel/main.go:26-36), without a GPU."""
from __future__ import annotations

import pytest

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200 import cli
from longbow_quarrel_b200.sampling import SamplingParams


def test_defaults_are_the_references():
    a = cli.parser().parse_args(["-model", "DIR"])
    assert (a.prompt, a.n, a.kv_cache_size) == ("Hello world", 20, 2048)
    assert (a.temp, a.topk, a.topp, a.penalty, a.stream) == (0.7, 40, 0.95, 1.1, False)
    assert (a.dtype, a.output, a.seed, a.batch) == ("bfloat16", "text", 0, 0)


def test_one_dash_or_two_as_with_go_flags():
    one = cli.parser().parse_args(["-model", "D", "-n", "5", "-temp", "0", "-topk", "3", "-topp", "0.5", "-penalty", "1.3",
                                   "-kv-cache-size", "512", "-stream"])
    two = cli.parser().parse_args(["--model", "D", "--n", "5", "--temp", "0", "--topk", "3", "--topp", "0.5", "--penalty",
                                   "1.3", "--kv-cache-size", "512", "--stream"])
    assert vars(one) == vars(two)
    assert (one.n, one.temp, one.topk, one.topp, one.penalty, one.kv_cache_size, one.stream) == (5, 0.0, 3, 0.5, 1.3, 512, True)
    with pytest.raises(SystemExit):
        cli.parser().parse_args(["-dtype", "float16"])


def test_the_model_comes_from_the_flag_or_the_variable(monkeypatch, capsys):
    monkeypatch.delenv("QUARREL_MODEL", raising=False)
    assert cli.main([]) == 1                                   # as the reference: an error and the usage
    assert "--model flag is required" in capsys.readouterr().err
    monkeypatch.setenv("QUARREL_MODEL", "/somewhere")
    assert cli.parser().parse_args([]).model == "/somewhere"


def test_prompts_as_ids_or_as_bytes_with_the_begin_token_in_front():
    p = cli.parser()
    a = p.parse_args(["-model", "D", "-prompt-ids", "1,15043, 3186 ; 7 8;"])
    assert cli._prompts(a, 32000, None) == [[1, 15043, 3186], [7, 8]]
    assert cli._prompts(a, 32000, 2) == [[2, 1, 15043, 3186], [2, 7, 8]]
    a = p.parse_args(["-model", "D", "-prompt-ids", "4", "-no-bos"])
    assert cli._prompts(a, 32000, 2) == [[4]]
    a = p.parse_args(["-model", "D", "-prompt", "hé"])
    assert cli._prompts(a, 200, None) == [[104, 195 % 200, 169]]   # UTF-8 bytes, folded into a small vocabulary


def test_options_reach_the_sampler_with_the_references_meanings():
    s = SamplingParams(temperature=0.0, top_k=40, top_p=0.95, repetition_penalty=1.1, seed=0)
    assert s.greedy and s.uses_history
    assert not SamplingParams(temperature=0.7).greedy
    assert not SamplingParams(repetition_penalty=1.0).uses_history
    assert SamplingParams(seed=5).resolved_seed() == 5
    assert SamplingParams(seed=0).resolved_seed() != 0         # seed 0: from the clock
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=0.0)


def test_prompts_from_a_file_and_synthetic_prompts(tmp_path):
    p = cli.parser()
    lines = tmp_path / "prompts.txt"
    lines.write_text("# two prompts\n1 15043 3186\n\n7, 8,9\n")
    a = p.parse_args(["-model", "D", "-prompt-file", str(lines)])
    assert cli._prompts(a, 32000, None) == [[1, 15043, 3186], [7, 8, 9]]
    assert cli._prompts(a, 32000, 2) == [[2, 1, 15043, 3186], [2, 7, 8, 9]]
    as_json = tmp_path / "prompts.json"
    as_json.write_text("[[4, 5], [6]]")
    assert cli.read_prompt_file(as_json) == [[4, 5], [6]]
    as_json.write_text("[4, 5, 6]")
    assert cli.read_prompt_file(as_json) == [[4, 5, 6]]
    lines.write_text("1 2\nthree\n")
    with pytest.raises(SystemExit, match="prompts.txt:2"):
        cli.read_prompt_file(lines)
    # synthetic prompts: -batch of them, -prompt-len ids each, drawn from -seed
    a = p.parse_args(["-model", "D", "-prompt-len", "12", "-batch", "3", "-seed", "5", "-no-bos"])
    got = cli._prompts(a, 100, 2)
    assert [len(q) for q in got] == [12, 12, 12] and all(0 <= t < 100 for q in got for t in q)
    assert got == cli._prompts(a, 100, 2) and got[0] != got[1]
    assert len(cli._prompts(p.parse_args(["-model", "D", "-prompt-len", "4"]), 100, None)) == 1


def test_the_bench_command_has_the_references_flags(monkeypatch, capsys):
    a = cli.bench_parser().parse_args(["-model", "DIR"])
    assert (a.prompt, a.tokens, a.output, a.timeout) == ("Hello world", 20, "text", 60)     # cmd/benchmark_json/main.go:28-35
    a = cli.bench_parser().parse_args(["--model", "DIR", "--tokens", "7", "--output", "json", "--timeout", "5",
                                       "-prompt-len", "128", "-batch", "8"])
    assert (a.tokens, a.output, a.timeout, a.prompt_len, a.batch) == (7, "json", 5, 128, 8)
    monkeypatch.delenv("QUARREL_MODEL", raising=False)
    assert cli.main(["bench"]) == 1
    assert "--model is required" in capsys.readouterr().err
