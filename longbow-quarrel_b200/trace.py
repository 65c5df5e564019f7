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
    args = ap.parse_args(argv)

    if not os.environ.get("HOME") or not os.access(os.environ["HOME"], os.W_OK):
        import tempfile
        os.environ["HOME"] = tempfile.mkdtemp(prefix="lq_home_")
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)

    import numpy as np
    import torch  # noqa: F401
    from longbow_quarrel_b200.engine import Engine

    engine = Engine.from_pretrained(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
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
            np.ascontiguousarray(arr).tofile(out / f"{step}.f32")
        for rid in obj.get("end", []):
            slot = slots.pop(str(rid), None)          # a request that never brought a token holds nothing
            if slot is not None:
                engine.end_sequence(slot)
        print(f"done {step}", flush=True)
    engine.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
