"""The command line, in the manner of the reference's `quarrel` binary.

Options keep the reference's names and meanings (cmd/quarrel/main_metal.go:24-36:
-model, -prompt, -n, -kv-cache-size, -temp, -topk, -topp, -penalty, -stream; from
cmd/benchmark_json/main.go:28-36: -output json; from cmd/generate_text/main.go:16-30: -v
and the QUARREL_MODEL variable).  Like Go's flag package, one or two dashes both work.
The model is a folder with config.json and model.safetensors instead of a GGUF file, and
a prompt is given as token ids, since the tokenizer is not part of this library; a text
prompt is read as its UTF-8 bytes.  As in the reference the begin-of-sequence token is put
in front of the prompt (cmd/quarrel/main_metal.go:113-114), when config.json names one.

    quarrel -model DIR -prompt-ids 1,2,3 -n 20
    quarrel -model DIR -prompt-file prompts.txt          one prompt a line (ids split by blanks or commas), or JSON
    quarrel -model DIR -prompt-len 128 -batch 8          seeded random prompts of 128 tokens, 8 at a time
    quarrel bench -model DIR -tokens 20 -output json     the reference's cmd/benchmark_json: greedy, its JSON fields

`bench` measures as cmd/benchmark_json/main.go:80-115 does: greedy sampling, the prefill duration up to the
first token, tokens a second over the tokens after the first, a timeout in seconds.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _flag(ap, name, **kw):
    ap.add_argument(f"-{name}", f"--{name}", **kw)


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="quarrel", description="Generate tokens with a Llama 3 model folder on one B200.")
    _flag(ap, "model", default=os.environ.get("QUARREL_MODEL", ""), help="model folder (config.json + model.safetensors)")
    _flag(ap, "random", default="", metavar="CONFIG.json", help="no folder: random weights for this config.json")
    _flag(ap, "prompt", default="Hello world", help="prompt text (read as UTF-8 bytes: there is no tokenizer)")
    _flag(ap, "prompt-ids", default="", help="prompt as token ids, e.g. 1,15043,3186; several prompts split by ';'")
    _flag(ap, "prompt-file", default="", metavar="FILE",
          help="prompts as token ids: one prompt a line (ids split by blanks or commas), or a JSON list of lists")
    _flag(ap, "prompt-len", type=int, default=0, metavar="N",
          help="no prompt given: random prompts of N token ids (drawn from -seed), as many as -batch says (default 1)")
    _flag(ap, "n", type=int, default=20, help="number of tokens to generate")
    _flag(ap, "kv-cache-size", type=int, default=2048, help="KV cache max sequence length")
    _flag(ap, "batch", type=int, default=0, help="sequences per batch (default: all prompts together)")
    _flag(ap, "temp", type=float, default=0.7, help="temperature for sampling (0 = greedy)")
    _flag(ap, "topk", type=int, default=40, help="top-K sampling")
    _flag(ap, "topp", type=float, default=0.95, help="top-P sampling")
    _flag(ap, "penalty", type=float, default=1.1, help="repetition penalty")
    _flag(ap, "seed", type=int, default=0, help="sampling seed (0 = from the clock)")
    _flag(ap, "stream", action="store_true", help="print tokens as they are generated")
    _flag(ap, "dtype", default="bfloat16", choices=["bfloat16", "float32"], help="precision of the whole model")
    _flag(ap, "output", default="text", choices=["text", "json"], help="output format")
    _flag(ap, "no-bos", action="store_true", help="do not put the begin-of-sequence token in front")
    _flag(ap, "convert-weights", action="store_true", help="round the stored weights to -dtype as they are loaded")
    _flag(ap, "allow-unexpected", action="store_true", help="tensors that the model does not name: a warning, not an error")
    _flag(ap, "v", action="store_true", help="verbose")
    return ap


def read_prompt_file(path) -> list[list[int]]:
    """Prompts as token ids: a JSON list of lists (or one list), or one prompt a line with the ids split by
    blanks or commas; empty lines and lines that start with # are skipped."""
    text = open(path).read()
    if text.lstrip().startswith("["):
        data = json.loads(text)
        if data and not isinstance(data[0], list):
            data = [data]
        return [[int(t) for t in p] for p in data]
    prompts = []
    for n, line in enumerate(text.splitlines(), 1):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        try:
            prompts.append([int(t) for t in line.replace(",", " ").split()])
        except ValueError:
            raise SystemExit(f"{path}:{n}: a prompt is token ids split by blanks or commas, found {line[:40]!r}") from None
    return prompts


def _prompts(args, vocab: int, bos) -> list[list[int]]:
    if args.prompt_file:
        prompts = read_prompt_file(args.prompt_file)
        if not prompts:
            raise SystemExit(f"{args.prompt_file}: no prompts")
    elif args.prompt_len > 0:
        import numpy as np
        rng = np.random.default_rng(args.seed)
        prompts = [[int(t) for t in rng.integers(0, vocab, args.prompt_len)] for _ in range(max(1, args.batch))]
    elif args.prompt_ids:
        prompts = [[int(t) for t in part.replace(",", " ").split()] for part in args.prompt_ids.split(";") if part.strip()]
    else:
        prompts = [[b % vocab for b in args.prompt.encode("utf-8")]]
    if bos is not None and not args.no_bos:
        prompts = [[bos] + p for p in prompts]
    return prompts


def bench_parser() -> argparse.ArgumentParser:
    """The flags of cmd/benchmark_json/main.go:28-36 (-model, -prompt, -tokens, -output, -timeout), and the
    ways of giving a prompt and a model that the main command has."""
    ap = argparse.ArgumentParser(prog="quarrel bench", description="Time greedy generation; print the reference's benchmark fields.")
    _flag(ap, "model", default=os.environ.get("QUARREL_MODEL", ""), help="model folder (config.json + model.safetensors)")
    _flag(ap, "random", default="", metavar="CONFIG.json", help="no folder: random weights for this config.json")
    _flag(ap, "prompt", default="Hello world", help="prompt text (read as UTF-8 bytes: there is no tokenizer)")
    _flag(ap, "prompt-ids", default="", help="prompt as token ids; several prompts split by ';'")
    _flag(ap, "prompt-file", default="", metavar="FILE", help="prompts as token ids, one a line or JSON")
    _flag(ap, "prompt-len", type=int, default=0, metavar="N", help="random prompts of N token ids, as many as -batch says")
    _flag(ap, "batch", type=int, default=0, help="sequences per batch (default: all prompts together)")
    _flag(ap, "tokens", type=int, default=20, help="number of tokens to generate")
    _flag(ap, "output", default="text", choices=["text", "json"], help="output format")
    _flag(ap, "timeout", type=int, default=60, help="timeout in seconds")
    _flag(ap, "kv-cache-size", type=int, default=0, help="KV cache max sequence length (default: what the prompts need)")
    _flag(ap, "seed", type=int, default=1, help="seed of random prompts and weights")
    _flag(ap, "dtype", default="bfloat16", choices=["bfloat16", "float32"], help="precision of the whole model")
    _flag(ap, "no-bos", action="store_true", help="do not put the begin-of-sequence token in front")
    _flag(ap, "convert-weights", action="store_true", help="round the stored weights to -dtype as they are loaded")
    _flag(ap, "allow-unexpected", action="store_true", help="tensors that the model does not name: a warning, not an error")
    return ap


class BenchTimeout(RuntimeError):
    pass


def _engine(args, data, prompts, n_new, batch, context):
    from .engine import Engine
    need = sorted((-(-(len(p) + n_new) // 64) * 64 for p in prompts), reverse=True)
    kw = dict(dtype=args.dtype, max_context=context, max_tokens=sum(need[:batch]), max_batch=batch)
    if args.random:
        return Engine.from_config(data, seed=args.seed or 1, **kw)
    return Engine.from_pretrained(args.model, convert_weights=args.convert_weights,
                                  unexpected="warn" if args.allow_unexpected else "error", **kw)


def bench_main(argv) -> int:
    args = bench_parser().parse_args(argv)
    if not args.model and not args.random:
        print("--model is required", file=sys.stderr)          # cmd/benchmark_json/main.go:37-39
        return 1
    from . import architectures  # noqa: F401  (registers the architectures)
    from .config import architecture_of, read_config_json
    from .sampling import SamplingParams
    data = json.loads(open(args.random).read()) if args.random else read_config_json(args.model)
    arch = architecture_of(data)
    spec = arch.describe(arch.config_from_dict(data))
    prompts = _prompts(args, spec.vocab_size, spec.bos_token)
    batch = args.batch or len(prompts)
    context = args.kv_cache_size or max(len(p) for p in prompts) + args.tokens
    engine = _engine(args, data, prompts, args.tokens, batch, context)
    start = time.perf_counter()
    first = [0.0]

    def on_token(i, tok):
        now = time.perf_counter()
        if not first[0]:
            first[0] = now                                      # the first token ends the prefill (main.go:72-77)
        if now - start > args.timeout:
            raise BenchTimeout(f"Inference timed out after {args.timeout} seconds")

    try:
        outputs = engine.generate(prompts, max_new_tokens=args.tokens, sampling=SamplingParams(temperature=0.0),
                                  stop_ids=[], callback=on_token, batch_size=args.batch or None)
    except BenchTimeout as e:
        print(str(e), file=sys.stderr)
        return 1
    total = time.perf_counter() - start
    prefill = (first[0] - start) if first[0] else 0.0
    gen = total - prefill if first[0] else 0.0
    n_tokens = sum(len(o) for o in outputs)
    # Tokens a second over the tokens after each sequence's first one (main.go:108-115).
    later = n_tokens - len(outputs)
    tps = later / gen if later > 0 and gen > 0 else (n_tokens / total if total > 0 else 0.0)
    result = {"throughput_tokens_per_sec": tps, "output": outputs, "total_duration_seconds": total,
              "prefill_duration_seconds": prefill, "generation_duration_seconds": gen, "tokens_generated": n_tokens}
    if args.output == "json":
        print(json.dumps(result))
    else:
        print(f"Throughput: {tps:.2f} tokens/sec")
        print(f"Prefill: {prefill:.3f}s  Generation: {gen:.3f}s  Total: {total:.3f}s  Tokens: {n_tokens}")
        for i, o in enumerate(outputs):
            print((f"[{i}] " if len(outputs) > 1 else "") + " ".join(str(t) for t in o))
    engine.close()
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "bench":
        return bench_main(argv[1:])
    args = parser().parse_args(argv)
    if not args.model and not args.random:
        print("Error: --model flag is required", file=sys.stderr)
        parser().print_usage(sys.stderr)
        return 1
    from . import architectures  # noqa: F401  (registers the architectures)
    from .sampling import SamplingParams
    from .config import architecture_of, read_config_json

    t_load = time.perf_counter()
    data = json.loads(open(args.random).read()) if args.random else read_config_json(args.model)
    arch = architecture_of(data)
    spec = arch.describe(arch.config_from_dict(data))
    prompts = _prompts(args, spec.vocab_size, spec.bos_token)
    batch = args.batch or len(prompts)
    # Room for the largest batch: every sequence's prompt and new tokens, in whole pages.
    engine = _engine(args, data, prompts, args.n, batch, args.kv_cache_size)
    load_s = time.perf_counter() - t_load
    if args.output == "text":
        print("=== Longbow-Quarrel B200 ===")
        print(f"Model: {args.model or args.random}")
        print(f"Architecture: {spec.name}  layers: {len(spec.layers)}  vocab: {spec.vocab_size}  dtype: {args.dtype}")
        if args.v:
            print(f"Loaded in {load_s:.2f}s; prompt tokens: {prompts}")

    def on_token(i, tok):
        if args.stream and args.output == "text":
            print(f"[{i}] {tok}" if len(prompts) > 1 else str(tok), flush=True)

    sampling = SamplingParams(temperature=args.temp, top_k=args.topk, top_p=args.topp,
                              repetition_penalty=args.penalty, seed=args.seed)
    t0 = time.perf_counter()
    outputs = engine.generate(prompts, max_new_tokens=args.n, sampling=sampling, callback=on_token,
                              batch_size=args.batch or None)
    total = time.perf_counter() - t0
    stats = engine.last_stats
    n_tokens = sum(len(o) for o in outputs)
    if args.output == "json":
        # The fields of cmd/benchmark_json/main.go:18-25.
        print(json.dumps({"throughput_tokens_per_sec": stats.decode_tokens_per_second, "output": outputs,
                          "total_duration_seconds": total, "prefill_duration_seconds": stats.prefill_seconds,
                          "generation_duration_seconds": stats.decode_seconds, "tokens_generated": n_tokens}))
    else:
        print(f"{n_tokens} tokens in {total:.3f}s ({n_tokens / total if total > 0 else 0.0:.2f} t/s)")
        for i, o in enumerate(outputs):
            print((f"[{i}] " if len(outputs) > 1 else "") + " ".join(str(t) for t in o))
    engine.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
