"""The command line, in the manner of the reference's `quarrel` binary.

Options keep the reference's names and meanings (cmd/quarrel/main_metal.go:24-36:
-model, -prompt, -n, -kv-cache-size, -temp, -topk, -topp, -penalty, -stream; from
cmd/benchmark_json/main.go:28-36: -output json; from cmd/generate_text/main.go:16-30: -v
and the QUARREL_MODEL variable).  Like Go's flag package, one or two dashes both work.
The model is a folder with config.json and model.safetensors instead of a GGUF file, and
a prompt is given as token ids, since the tokenizer is not part of this library; a text
prompt is read as its UTF-8 bytes.  As in the reference the begin-of-sequence token is put
in front of the prompt (cmd/quarrel/main_metal.go:113-114), when config.json names one.
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
    _flag(ap, "v", action="store_true", help="verbose")
    return ap


def _prompts(args, vocab: int, bos) -> list[list[int]]:
    if args.prompt_ids:
        prompts = [[int(t) for t in part.replace(",", " ").split()] for part in args.prompt_ids.split(";") if part.strip()]
    else:
        prompts = [[b % vocab for b in args.prompt.encode("utf-8")]]
    if bos is not None and not args.no_bos:
        prompts = [[bos] + p for p in prompts]
    return prompts


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    if not args.model and not args.random:
        print("Error: --model flag is required", file=sys.stderr)
        parser().print_usage(sys.stderr)
        return 1
    from .engine import Engine
    from .sampling import SamplingParams
    from .config import architecture_of, read_config_json

    t_load = time.perf_counter()
    data = json.loads(open(args.random).read()) if args.random else read_config_json(args.model)
    arch = architecture_of(data)
    spec = arch.describe(arch.config_from_dict(data))
    prompts = _prompts(args, spec.vocab_size, spec.bos_token)
    batch = args.batch or len(prompts)
    # Room for the largest batch: every sequence's prompt and new tokens, in whole pages.
    need = sorted((-(-(len(p) + args.n) // 64) * 64 for p in prompts), reverse=True)
    kw = dict(dtype=args.dtype, max_context=args.kv_cache_size, max_tokens=sum(need[:batch]), max_batch=batch)
    if args.random:
        engine = Engine.from_config(data, seed=args.seed or 1, **kw)
    else:
        engine = Engine.from_pretrained(args.model, **kw)
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
