"""Measurement: decoded tokens a second of a Llama-3.1-8B-shaped model with random
bfloat16 weights on one B200, with prefill throughput, the decode step's fraction of the
HBM roofline, decode at batch 1 and 64, and the other workloads that the baseline names
(the Llama-3.2-3B and -1B shapes, the two tiny configurations on the CPU's plain implementation).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  The timed
region is K steps bracketed by CUDA events after W untimed steps; every step reads all
layer weights (about 15 GB, far more than the 126 MB L2), so no L2 flush is needed.

How generation is timed follows the reference's own benchmark (cmd/benchmark_json/main.go:80-86,
108-115): the prompt step up to the first token is the prefill, tokens a second are counted over the
tokens after the first.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def llama(hidden, layers, heads, kv_heads, head_dim, inter, factor, tied):
    return dict(architectures=["LlamaForCausalLM"], hidden_size=hidden, num_hidden_layers=layers,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                vocab_size=128256, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=tied, max_position_embeddings=131072)


MODEL = llama(4096, 32, 32, 8, 128, 14336, 8.0, False)           # Llama 3.1 8B layer sizes: the headline
MODEL_3B = llama(3072, 28, 24, 8, 128, 8192, 32.0, True)         # Llama 3.2 3B
MODEL_1B = llama(2048, 16, 32, 8, 64, 8192, 32.0, True)          # Llama 3.2 1B
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
E2E_WARM = 48          # decode steps after a prompt step before a decode figure is timed (device-timed or end to end)
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


class FastClocks:
    """SM clock read through NVML every few milliseconds (reading only), to set the duration of single
    decode steps against the clock they ran at."""

    def __init__(self, period_s: float = 0.004):
        self.period, self.samples, self._stop, self._thread, self._nvml = period_s, [], threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml, self._handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(0)
        except Exception:
            self._nvml = None

    def start(self):
        if self._nvml is None:
            return
        def run():
            nv = self._nvml
            while not self._stop.is_set():
                try:
                    self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                except Exception:
                    return
                self._stop.wait(self.period)
        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def median_between(self, t0: float, t1: float):
        mhz = [m for t, m in self.samples if t0 <= t <= t1]
        return statistics.median(mhz) if mhz else None


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


def prefill_flops(cfg, layers: int, lengths, logit_rows: int) -> float:
    tokens = sum(lengths)
    matmul = 2.0 * tokens * layers * linear_params(cfg) + 2.0 * logit_rows * cfg["vocab_size"] * cfg["hidden_size"]
    attn = sum(layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * n * (n + 1) / 2.0 for n in lengths)
    return matmul + attn


def events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def decode_run(torch, engine, rng, V, batch: int, steps: int, warm: int, prompt_len: int, params, sampler=None,
               settle: int = 0):
    """One prompt step, then decode steps fed with token ids that were drawn beforehand (no host read in the
    loop), each followed by the sampler on its logits: what the device does in a step, timed on the device.
    settle: untimed decode steps before the `warm` warm-up steps, for the clocks to come back from the prompt
    step (a long prompt step runs at the power cap, and the steps right after it at about half the clock)."""
    from longbow_quarrel_b200.kernels import ops
    from longbow_quarrel_b200.sampling import sample
    slots = [engine.new_sequence() for _ in range(batch)]
    prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(batch)]
    logits = engine.step(list(zip(slots, prompts)))
    warm += settle
    feed = rng.integers(0, V, (warm + steps, batch))
    scratch = torch.empty_like(logits)
    seq_ids = torch.arange(batch, dtype=torch.int32, device=logits.device)
    step_ids = torch.zeros(batch, dtype=torch.int32, device=logits.device)

    def one(i):
        out = engine.step([(s, [int(t)]) for s, t in zip(slots, feed[i])])
        sample(out, params, 1, seq_ids, step_ids, scratch=scratch)
    for i in range(warm):
        one(i)
    before = ops.launch_count()
    a, b = events(torch)
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    a.record()
    for i in range(warm, warm + steps):
        one(i)
    b.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = a.elapsed_time(b)
    for s in slots:
        engine.end_sequence(s)
    mean_ctx = prompt_len + warm + (steps - 1) / 2.0 + 1
    return ms, mean_ctx, ops.launch_count() - before, clocks


def timed_generate(engine, prompts, n_new, params, batch):
    """engine.generate with the arrival time of every step's tokens on the host: [t_prompt_done, t_1, ...]."""
    times, calls = [], [0]
    t0 = time.perf_counter()

    def on_token(i, tok):
        if calls[0] % batch == 0:
            times.append(time.perf_counter())
        calls[0] += 1
    out = engine.generate(prompts, max_new_tokens=n_new, sampling=params, stop_ids=[], callback=on_token)
    return out, t0, times


def other_workload(torch, np, peaks, name, cfg, prompt_lengths, n_steps, params, device_steps):
    """A workload of the baseline through the public entry point: one batch of prompts, then n_steps decode
    steps, host tokens in and out.  Returns flat figures for `points`."""
    from longbow_quarrel_b200.engine import Engine
    rng = np.random.default_rng(1)
    V, L, B = cfg["vocab_size"], cfg["num_hidden_layers"], len(prompt_lengths)
    longest = max(prompt_lengths) + n_steps + 1
    tokens = sum(-(-(n + n_steps + 1) // 64) * 64 for n in prompt_lengths)
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=tokens, max_batch=B, max_context=longest,
                                gain_std=0.0)
    prompts = [rng.integers(0, V, n).tolist() for n in prompt_lengths]
    engine.generate(prompts, max_new_tokens=4, sampling=params, stop_ids=[])           # warm-up: kernels, graphs
    torch.cuda.synchronize()
    _, t0, times = timed_generate(engine, prompts, n_steps + 1, params, B)
    prefill_s = times[0] - t0
    decode_s = times[-1] - times[0]
    steps = len(times) - 1
    ms_step = decode_s / steps * 1e3
    mean_ctx = sum(prompt_lengths) / B + (steps + 1) / 2.0
    achieved = decode_bytes(cfg, L, B, mean_ctx) / (ms_step / 1e3) / 1e9
    out = {f"{name}_decode": B * steps / decode_s, f"{name}_ms_per_step": ms_step, f"{name}_decode_frac": achieved / peaks["hbm_gbs"],
           f"{name}_prefill": sum(prompt_lengths) / prefill_s,
           f"{name}_prefill_frac": prefill_flops(cfg, L, prompt_lengths, B) / prefill_s / (peaks["bf16_tflops"] * 1e12)}
    if device_steps:
        # The same decode steps without the host in the loop (tokens drawn beforehand, nothing read back): what is
        # left of a step when the host costs nothing.  1 - device / end-to-end is the host's share of a step.
        # (at the same mean context as the steps above: the prompt is as much longer as those steps are more)
        start = max(1, int(mean_ctx - E2E_WARM - 8 - device_steps / 2.0))
        ms, _, _, _ = decode_run(torch, engine, rng, V, B, device_steps, 8, start, params, settle=E2E_WARM)
        out[f"{name}_device_ms_per_step"] = ms / device_steps
        out[f"{name}_host_share"] = max(0.0, 1.0 - (ms / device_steps) / ms_step)
    engine.close()
    del engine
    torch.cuda.empty_cache()
    return out


def tiny_workloads(torch) -> dict:
    """The two tiny configurations of the baseline (float32): seconds of the plain CPU implementation (the
    oracle of the tests, whole sequences re-run for every token) and of the engine's 32-bit path on the GPU for
    the same greedy generation, and whether they chose the same tokens."""
    import tempfile

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_llama
    from helpers import TINY, make_model_folder, random_tokens
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.sampling import SamplingParams
    out = {}
    for name, lengths, n_new in (("a", [7, 3, 12, 1], 8), ("b", [20, 5, 33], 16)):
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_model_folder(tmp, name.upper(), seed=7)
            vocab = TINY[name.upper()]["vocab_size"]
            prompts = [random_tokens(n, vocab, 300 + i) for i, n in enumerate(lengths)]
            cfg, weights = plain_llama.load_folder(folder)
            t0 = time.perf_counter()
            want = [plain_llama.greedy(cfg, weights, p, n_new) for p in prompts]
            out[f"tiny_{name}_plain_cpu_s"] = time.perf_counter() - t0
            engine = Engine.from_pretrained(folder, dtype="float32", max_tokens=1024)
            engine.generate(prompts, max_new_tokens=2, sampling=SamplingParams(), stop_ids=[])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = engine.generate(prompts, max_new_tokens=n_new, sampling=SamplingParams(), stop_ids=[])
            out[f"tiny_{name}_engine_fp32_s"] = time.perf_counter() - t0
            out[f"tiny_{name}_same_tokens"] = got == want
            engine.close()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                    help="fewer layers than the model has (reported in config)")
    ap.add_argument("--no-points", action="store_true", help="only the headline: no other batches, models or tiny runs")
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
    from longbow_quarrel_b200.sampling import SamplingParams

    peaks, peaks_from = load_peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    L = args.layers
    max_batch = BATCH if args.no_points else 64
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * CONTEXT, max_batch=max_batch,
                                max_context=CONTEXT, gain_std=0.0)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    greedy = SamplingParams(temperature=0.0)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    def prefill_once():
        slot = engine.new_sequence()
        toks = rng.integers(0, V, PREFILL_TOKENS).tolist()
        a, b = events(torch)
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
    pf_flops = prefill_flops(cfg, L, [PREFILL_TOKENS], 1)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ------------------------------------------------------------------ decode, timed on the device
    ms, mean_ctx, launches, clocks = decode_run(torch, engine, rng, V, BATCH, K, W, CONTEXT - (W + K + E2E_WARM), greedy,
                                                ClockSampler(), settle=E2E_WARM)
    ms_per_step = ms / K
    value = BATCH * K / (ms / 1e3)
    bytes_step = decode_bytes(cfg, L, BATCH, mean_ctx)
    achieved = bytes_step / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peaks_from}

    # ------------------------------------------------------------------ end to end through generate()
    # K steps through the public entry point: host token ids in, one copy of the step's integers to the device and
    # one read of the sampled ids a step.  Timed on the host from the arrival of one step's tokens to that of the
    # K-th step after it.  The decode steps right after a long prompt step run at the reduced clocks that the
    # prompt step under the power cap leaves behind (about a dozen steps; reported below with the clock they ran
    # at), so this figure, like the device-timed one above, begins E2E_WARM + W steps after the prompt.
    W_dev, W = W, W + E2E_WARM
    prompt_len = CONTEXT - (W + K) - 1
    prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(BATCH)]
    engine.generate(prompts[:BATCH], max_new_tokens=3, sampling=greedy, stop_ids=[])       # warm-up
    fast = FastClocks()
    fast.start()
    _, t0, times = timed_generate(engine, prompts, W + K + 1, greedy, BATCH)
    fast.stop()
    from longbow_quarrel_b200.engine.step import pack_step
    flat_bytes = pack_step([(i, [0]) for i in range(BATCH)], None, [0] * BATCH, engine.stepper.needs)[0].nbytes   # a step's integers
    e2e_s = times[W + K] - times[W]
    # The first steps after a prompt step against the steady ones, each with the clock it ran at: if duration x
    # clock is the same, the longer first steps are the device's clocks coming back up, not the host.
    head = min(10, W)
    head_ms = (times[head] - times[0]) / head * 1e3
    steady_ms = e2e_s / K * 1e3
    head_mhz, steady_mhz = fast.median_between(times[0], times[head]), fast.median_between(times[W], times[W + K])
    e2e = {"value": BATCH * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": flat_bytes, "d2h_bytes_per_step": 4 * BATCH,
           "steps": K, "after_warmup_steps": W, "ms_per_step": steady_ms, "sm_mhz": steady_mhz,
           "first_steps_after_prompt": {"steps": head, "ms_per_step": head_ms, "sm_mhz": head_mhz},
           "from_first_token": {"value": BATCH * (W + K) / (times[W + K] - times[0]), "steps": W + K}}

    W = W_dev
    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = max(16, K // 2)
            ms_b, ctx_b, _, _ = decode_run(torch, engine, rng, V, b, k, W, CONTEXT - (W + k + E2E_WARM), greedy, settle=E2E_WARM)
            points[f"decode_b{b}"] = b * k / (ms_b / 1e3)
            points[f"decode_b{b}_frac"] = decode_bytes(cfg, L, b, ctx_b) / (ms_b / k / 1e3) / 1e9 / peaks["hbm_gbs"]
    engine.close()
    del engine
    torch.cuda.empty_cache()
    if not args.no_points:
        # Llama-3.2-3B shape: 16 unequal prompts U[1, 2048], then 256 decode steps (greedy).
        lengths = [int(n) for n in np.random.default_rng(2).integers(1, 2049, 16)]
        points.update(other_workload(torch, np, peaks, "llama32_3b", MODEL_3B, lengths, 256, greedy, 0))
        # Llama-3.2-1B shape: batch 64, prompts of 128, 1,024 decode steps at temperature 1.
        points.update(other_workload(torch, np, peaks, "llama32_1b", MODEL_1B, [128] * 64, 1024,
                                     SamplingParams(temperature=1.0, seed=5), 256))
        points.update(tiny_workloads(torch))

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
                   "decode_context_mean": mean_ctx, "prefill_tokens": PREFILL_TOKENS, "settle_steps_after_prompt": E2E_WARM,
                   "l2": "every step reads 15 GB of weights, far more than L2; no flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
