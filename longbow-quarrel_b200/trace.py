"""Trace replay: given token ids go through the model step by step, logits come out.

It samples nothing.  It drives the engine that generation uses -- the same model,
step function, cache and kernels -- and has no forward pass, cache or loader of
its own.  The reference's seeds for it are cmd/debug_layers/main.go:87-131 (fixed
prompts, one greedy token each), cmd/debug_generation/main.go:61-93 (token by
token) and InferWithCallbackLogits (internal/engine/engine.go:1287-1290).

Standard input carries one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` gives each request's next tokens and the places among them whose logits
are wanted; `end` names requests that are finished after the step.  For a step in
which something is wanted, OUT/<step>.f32 receives float32 little-endian
[wanted, vocab] in the order of the entries and of `want`.  After every step a
line `done <step>` is printed and flushed.

Two optional looks inside, for finding the layer or the kernel where two runs part
(the reference's activation trace, internal/engine/types.go:308-323, is the seed):
`--layer-stats` also writes OUT/<step>.layers.f32, float32 [wanted, runs + 1]: the root
mean square of each wanted row of the residual stream after the embedding and after
every run of a layer; `--kernel-counts` writes OUT/kernels.json when the input ends:
how often each kernel launcher (and each path inside it) ran.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--layer-stats", action="store_true",
                    help="also write <step>.layers.f32: RMS of the residual stream of each wanted row after every layer")
    ap.add_argument("--kernel-counts", action="store_true", help="write kernels.json: launches by kernel, at the end")
    args = ap.parse_args(argv)

    if not os.environ.get("HOME") or not os.access(os.environ["HOME"], os.W_OK):
        import tempfile
        os.environ["HOME"] = tempfile.mkdtemp(prefix="lq_home_")
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)

    import numpy as np
    import torch
    from longbow_quarrel_b200.engine import Engine

    engine = Engine.from_pretrained(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
    layer_rms: list = []
    if args.layer_stats:
        def probe(run, x, ctx):
            if ctx.want_rows is not None:
                rows = x[ctx.want_rows.long()]
                layer_rms.append(rows.double().pow(2).mean(dim=1).sqrt().float())
        engine.model.probe = probe
    slots: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries, want = [], []
        for e in obj["entries"]:
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_sequence()
            entries.append((slots[rid], e["tokens"]))
            want.append(e.get("want", []))
        logits = engine.step(entries, want) if entries else None      # a step may only end requests
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            engine.check()
            np.ascontiguousarray(arr).tofile(out / f"{step}.f32")
            if layer_rms:
                torch.stack(layer_rms, dim=1).to("cpu").numpy().astype("<f4").tofile(out / f"{step}.layers.f32")
        layer_rms.clear()
        for rid in obj.get("end", []):
            slot = slots.pop(str(rid), None)          # a request that never brought a token holds nothing
            if slot is not None:
                engine.end_sequence(slot)
        print(f"done {step}", flush=True)
    if args.kernel_counts:
        from longbow_quarrel_b200.kernels import ops
        (out / "kernels.json").write_text(json.dumps(ops.launches_by_name(), indent=1, sort_keys=True))
    engine.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
