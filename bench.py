"""Measurement: decoded tokens a second of a Llama-3.1-8B-shaped model with random
bfloat16 weights on one B200, with prefill throughput, the decode step's fraction of the
HBM roofline, and decode at batch 1 and 64.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  The timed
region is K steps bracketed by CUDA events after W untimed steps; every step reads all
layer weights (about 15 GB, far more than the 126 MB L2), so no L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Llama 3.1 8B layer sizes.
MODEL = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
             rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192),
             rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=131072)
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

REFERENCE_UNAVAILABLE = ("the reference is a Go program for Apple Metal with no Python package: pip reports "
                         "\"Directory is not installable. Neither 'setup.py' nor 'pyproject.toml' found\", "
                         "and no Go toolchain or Metal exists here")


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            peaks = {k: float(data[k]) for k in FALLBACK_PEAKS if k in data}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={','.join(self.FIELDS)}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != len(self.FIELDS):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def linear_params(cfg) -> int:
    D, H, Hkv, hd, F = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"])
    return (H + 2 * Hkv) * hd * D + H * hd * D + 3 * F * D


def decode_bytes(cfg, layers: int, batch: int, context: float) -> float:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    weights = 2.0 * (layers * linear_params(cfg) + cfg["vocab_size"] * cfg["hidden_size"])
    weights += 4.0 * (2 * layers + 1) * cfg["hidden_size"]            # norm gains (float32)
    kv = batch * context * layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2.0
    return weights + kv


def prefill_flops(cfg, layers: int, tokens: int, logit_rows: int) -> float:
    matmul = 2.0 * tokens * layers * linear_params(cfg) + 2.0 * logit_rows * cfg["vocab_size"] * cfg["hidden_size"]
    attn = layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2.0
    return matmul + attn


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                    help="fewer layers than the model has (reported in config)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a one-GPU library: --gpus {args.gpus} is not supported, run it with --gpus 1")
        return 2
    K, W = args.steps, max(3, args.warmup)

    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.kernels import ops
    from longbow_quarrel_b200.sampling import SamplingParams, sample

    peaks, peaks_from = load_peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    L = args.layers
    max_batch = BATCH if args.no_points else 64
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * CONTEXT, max_batch=max_batch,
                                max_context=CONTEXT, gain_std=0.0)
    dev = engine.device
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    greedy = SamplingParams(temperature=0.0)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    def prefill_once():
        slot = engine.new_sequence()
        toks = rng.integers(0, V, PREFILL_TOKENS).tolist()
        a, b = events()
        torch.cuda.synchronize()
        a.record()
        engine.step([(slot, toks)])
        b.record()
        torch.cuda.synchronize()
        engine.end_sequence(slot)
        return a.elapsed_time(b)
    for _ in range(3):
        prefill_once()
    prefill_ms = statistics.median(prefill_once() for _ in range(5))
    pf_flops = prefill_flops(cfg, L, PREFILL_TOKENS, 1)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ------------------------------------------------------------------ decode, timed on the device
    def decode_run(batch: int, steps: int, warm: int, sampler: ClockSampler | None = None):
        """Prompts that leave room for warm + steps tokens in the context, one prefill step, then
        decode steps fed with token ids that were drawn beforehand (no host read in the loop)."""
        prompt_len = CONTEXT - (warm + steps)
        slots = [engine.new_sequence() for _ in range(batch)]
        prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(batch)]
        logits = engine.step(list(zip(slots, prompts)))
        feed = rng.integers(0, V, (warm + steps, batch))
        scratch = torch.empty_like(logits)
        for i in range(warm):
            logits = engine.step([(s, [int(t)]) for s, t in zip(slots, feed[i])])
            sample(logits, greedy, 0, scratch=scratch)
        before = ops.launch_count()
        a, b = events()
        torch.cuda.synchronize()
        if sampler:
            sampler.start()
        a.record()
        for i in range(warm, warm + steps):
            logits = engine.step([(s, [int(t)]) for s, t in zip(slots, feed[i])])
            sample(logits, greedy, 0, scratch=scratch)
        b.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        ms = a.elapsed_time(b)
        for s in slots:
            engine.end_sequence(s)
        mean_ctx = prompt_len + warm + (steps - 1) / 2.0 + 1
        return ms, mean_ctx, ops.launch_count() - before, clocks

    ms, mean_ctx, launches, clocks = decode_run(BATCH, K, W, ClockSampler())
    ms_per_step = ms / K
    value = BATCH * K / (ms / 1e3)
    bytes_step = decode_bytes(cfg, L, BATCH, mean_ctx)
    achieved = bytes_step / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peaks_from}

    # ------------------------------------------------------------------ end to end through generate()
    prompt_len = CONTEXT - (W + K)
    prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(BATCH)]
    engine.generate(prompts[:BATCH], max_new_tokens=3, sampling=greedy, stop_ids=[])       # warm-up
    engine.generate(prompts, max_new_tokens=K + 1, sampling=greedy, stop_ids=[])
    st = engine.last_stats
    flat_bytes = 4 * (3 * BATCH + 2 * BATCH + (BATCH + 1) + BATCH + 7 * 3)       # the step's integers, padded parts
    e2e = {"value": BATCH * st.decode_steps / st.decode_seconds, "unit": "tokens/s",
           "h2d_bytes_per_step": flat_bytes, "d2h_bytes_per_step": 4 * BATCH}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = max(16, K // 2)
            ms_b, _, _, _ = decode_run(b, k, W)
            points[f"decode_b{b}"] = b * k / (ms_b / 1e3)

    line = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, batch 8, context 4096", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random bf16 weights N(0, 0.02), uniform random token ids",
        "config": {"model": "Llama-3.1-8B shape", "global_batch": BATCH, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "layers": L, "layers_of_model": MODEL["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
                   "vocab_size": V, "rope_theta": cfg["rope_theta"], "rope_scaling": "llama3 factor 8 low 1 high 4 orig 8192",
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied_embeddings": False,
                   "decode_context_mean": mean_ctx, "prefill_tokens": PREFILL_TOKENS,
                   "l2": "every step reads 15 GB of weights, far more than L2; no flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
