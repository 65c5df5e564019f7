"""Timing single kernels and single steps, for roofline work and for profilers.

    python -m longbow_quarrel_b200.kernels.microbench gemm_tc --m 64 --n 28672 --k 4096 --epi swiglu
    python -m longbow_quarrel_b200.kernels.microbench gemm_tc --m 2048 --n 6144 --k 4096
    python -m longbow_quarrel_b200.kernels.microbench attn_decode --batch 8 --context 4096
    python -m longbow_quarrel_b200.kernels.microbench attn_prefill --tokens 2048
    python -m longbow_quarrel_b200.kernels.microbench step --batch 8 --context 4096 --layers 4
    python -m longbow_quarrel_b200.kernels.microbench prefill --tokens 2048 --layers 4
    python -m longbow_quarrel_b200.kernels.microbench timeline --batch 8 --layers 6
    python -m longbow_quarrel_b200.kernels.microbench timeline --prompt --tokens 2048 --layers 4
    python -m longbow_quarrel_b200.kernels.microbench sample --batch 64 --temperature 0.7 --top-k 40 --top-p 0.95

Each kernel is timed with CUDA events over `--iters` launches after `--warmup`, captured
into one CUDA graph so that no host time lies between the launches (`--no-graph` launches
them from the host one by one); operands are rotated through enough copies to exceed the
126 MB L2, so every launch reads from HBM.  One JSON line is printed: time, bytes or flops moved, achieved GB/s and TFLOP/s.
`step` builds a model of Llama-3.1-8B layer sizes with `--layers` layers, fills the cache
of `--batch` sequences to `--context` tokens with random keys and values (no prefill),
and runs decode steps; with `--eager` the step's kernels are launched one by one instead
of replaying a captured graph, which is what a launch-by-launch profile wants.
`timeline` runs the same steps as captured graphs under the CUDA activity records of
torch.profiler and prints, for each kind of kernel of the last step, how long it ran and how
much later it ended than the kernel before it (kernels overlap through programmatic dependent
launch, so the second number is what a kernel adds to the step).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

L2_BYTES = 126 * 1024 * 1024
EPIS = {"bf16": 0, "f32": 1, "resid": 2, "swiglu": 3}


GRAPH = True      # time kernels as one captured graph of `iters` launches: no host time between them


def _time(fn, iters: int, warmup: int, graph: bool | None = None) -> float:
    for i in range(warmup):
        fn(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if GRAPH if graph is None else graph:
        g = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), torch.cuda.graph(g, stream=stream):
            for i in range(iters):
                fn(warmup + i)
        torch.cuda.current_stream().wait_stream(stream)
        g.replay()
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters
    a.record()
    for i in range(iters):
        fn(warmup + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def _copies(nbytes: int) -> int:
    return max(2, -(-2 * L2_BYTES // max(nbytes, 1)))


def bench_gemm(kind: str, args) -> dict:
    from . import ops
    M, N, K, epi = args.m, args.n, args.k, EPIS[args.epi]
    dev = "cuda"
    n = min(_copies(N * K * 2), 64)
    ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(n)]
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(n)]
    res = torch.zeros(M, N, device=dev, dtype=torch.float32) if args.epi == "resid" else None
    fn = {"gemm_skinny": ops.gemm_skinny, "gemm_tc": ops.gemm_tc}[kind]
    outs = {}

    def run(i):
        outs["o"] = fn(xs[i % n], ws[i % n], epi, res)
    ms = _time(run, args.iters, args.warmup)
    out_bytes = outs["o"].numel() * outs["o"].element_size() * (2 if args.epi == "resid" else 1)
    nbytes = N * K * 2 + M * K * 2 + out_bytes
    flops = 2.0 * M * N * K
    return {"kernel": kind, "M": M, "N": N, "K": K, "epi": args.epi, "ms": ms, "bytes": nbytes,
            "gbs": nbytes / ms / 1e6, "tflops": flops / ms / 1e9, "weight_copies": n}


def bench_chain(args) -> dict:
    """The four products of a decoder layer one after another (no attention between them), over
    several layers' weights, each product naming the weights that follow it."""
    from . import ops
    from .linear import interleave_gate_up
    M, D, F, dev = args.m, 4096, 14336, "cuda"
    L = max(2, args.layers)
    mk = lambda n, k: torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02
    layers = [dict(qkv=mk(6144, D), o=mk(D, D), gu=interleave_gate_up(mk(F, D), mk(F, D)), down=mk(D, F)) for _ in range(L)]
    x = torch.randn(M, D, device=dev, dtype=torch.bfloat16)
    res = torch.zeros(M, D, device=dev, dtype=torch.float32)

    gain = torch.ones(D, device=dev, dtype=torch.float32)
    attn = torch.randn(M, D, device=dev, dtype=torch.bfloat16)

    def run(i):
        rows = x
        for j, w in enumerate(layers):
            nxt = layers[(j + 1) % L]
            ops.gemm_skinny(rows, w["qkv"], ops.EPI_BF16, next_w=w["o"])
            _, h2 = ops.gemm_skinny(attn, w["o"], ops.EPI_RESID, res, emit=(gain, 1e-5), next_w=w["gu"])
            act = ops.gemm_skinny(h2, w["gu"], ops.EPI_SWIGLU, next_w=w["down"])
            _, rows = ops.gemm_skinny(act, w["down"], ops.EPI_RESID, res, emit=(gain, 1e-5), next_w=nxt["qkv"])
    ms = _time(run, args.iters, args.warmup)
    nbytes = L * (6144 * D + D * D + 2 * F * D + D * F) * 2
    return {"kernel": "chain of a layer's products", "M": M, "layers": L, "ms_per_layer": ms / L, "gbs": nbytes / ms / 1e6,
            "prefetch_bytes": ops.PREFETCH_BYTES}


def bench_sample(args) -> dict:
    """The sampler on --batch rows of --vocab logits (rotated through copies larger than L2)."""
    from ..sampling import SamplingParams, sample
    rows, V, dev = args.batch, args.vocab, "cuda"
    n = min(_copies(rows * V * 4), 64)
    logits = [torch.randn(rows, V, device=dev) * 3 for _ in range(n)]
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=3)
    seq = torch.arange(rows, dtype=torch.int32, device=dev)
    step = torch.zeros(rows, dtype=torch.int32, device=dev)
    scratch = torch.empty_like(logits[0]) if args.one_block else None
    out = torch.empty(rows, dtype=torch.int32, device=dev)

    def run(i):
        sample(logits[i % n], params, 3, seq, step, scratch=scratch, out=out, step_offset=i, one_block=args.one_block)
    ms = _time(run, args.iters, args.warmup)
    nbytes = rows * V * 4
    return {"kernel": "sample (one block a row)" if args.one_block else "sample (a cluster a row)", "rows": rows, "vocab": V,
            "temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p, "ms": ms, "bytes": nbytes,
            "gbs": nbytes / ms / 1e6}


def _paged(batch: int, context: int, Hkv: int, hd: int, dev):
    pages_per = -(-context // 64)
    n_pages = batch * pages_per
    k = torch.randn(n_pages, Hkv, 64, hd, device=dev, dtype=torch.bfloat16)
    v = torch.randn(n_pages, Hkv, 64, hd, device=dev, dtype=torch.bfloat16)
    table = torch.randperm(n_pages, device=dev).to(torch.int32).reshape(batch, pages_per).contiguous()
    return k, v, table


def bench_attn_decode(args) -> dict:
    from . import attention, ops
    B, C, H, Hkv, hd = args.batch, args.context, args.heads, args.kv_heads, args.head_dim
    dev = "cuda"
    n = min(_copies(B * C * Hkv * hd * 4), 16)
    caches = [_paged(B, C, Hkv, hd, dev) for _ in range(n)]
    q = torch.randn(B, (H + 2 * Hkv) * hd, device=dev, dtype=torch.bfloat16)
    pos = torch.full((B,), C - 1, dtype=torch.int32, device=dev)
    seq = torch.arange(B, dtype=torch.int32, device=dev)
    splits = args.splits or attention.decode_splits(B, Hkv, -(-(H // Hkv) // 16), C, attention.resident_blocks('cuda'))

    def run(i):
        k, v, table = caches[i % n]
        ops.attn_decode(q, k, v, table, pos, seq, seq, H, Hkv, hd, 64, hd ** -0.5, None, splits)
    ms = _time(run, args.iters, args.warmup)
    nbytes = B * C * Hkv * hd * 2 * 2
    return {"kernel": "attn_decode", "batch": B, "context": C, "heads": H, "kv_heads": Hkv, "head_dim": hd,
            "splits": splits, "ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6}


def bench_attn_prefill(args) -> dict:
    from . import ops
    T, H, Hkv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
    dev = "cuda"
    k, v, table = _paged(1, T, Hkv, hd, dev)
    q = torch.randn(T, (H + 2 * Hkv) * hd, device=dev, dtype=torch.bfloat16)
    nb = -(-T // 64)
    starts = torch.arange(nb - 1, -1, -1, dtype=torch.int32, device=dev) * 64
    blocks = (torch.zeros(nb, dtype=torch.int32, device=dev), starts.contiguous(),
              torch.minimum(torch.full_like(starts, 64), T - starts).contiguous(), starts.clone())
    slots = torch.zeros(1, dtype=torch.int32, device=dev)
    kv_len = torch.full((1,), T, dtype=torch.int32, device=dev)

    nb2 = -(-T // 128)
    starts2 = torch.arange(nb2 - 1, -1, -1, dtype=torch.int32, device=dev) * 128
    blocks128 = (torch.zeros(nb2, dtype=torch.int32, device=dev), starts2.contiguous(),
                 torch.minimum(torch.full_like(starts2, 128), T - starts2).contiguous(), starts2.clone())
    tc = args.what == "attn_prefill_tc"

    def run(i):
        if tc:
            ops.attn_prefill_tc(q, k, v, table, slots, kv_len, blocks128, H, Hkv, hd, 64, hd ** -0.5, None)
        else:
            ops.attn_prefill(q, k, v, table, slots, kv_len, blocks, H, Hkv, hd, 64, hd ** -0.5, None)
    ms = _time(run, args.iters, args.warmup)
    flops = 4.0 * H * hd * T * (T + 1) / 2.0
    return {"kernel": args.what, "tokens": T, "heads": H, "kv_heads": Hkv, "head_dim": hd, "ms": ms,
            "tflops": flops / ms / 1e9}


# Layer sizes of the three Llama 3 shapes that the measurements name: hidden, heads, kv heads, head_dim, intermediate, tied.
SHAPES = {"8b": (4096, 32, 8, 128, 14336, False), "3b": (3072, 24, 8, 128, 8192, True), "1b": (2048, 32, 8, 64, 8192, True)}


def _config(args) -> dict:
    D, H, Hkv, hd, F, tied = SHAPES[args.shape]
    return dict(architectures=["LlamaForCausalLM"], hidden_size=D, num_hidden_layers=args.layers,
                num_attention_heads=H, num_key_value_heads=Hkv, head_dim=hd, intermediate_size=F,
                vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=131072,
                tie_word_embeddings=tied,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))


def _decode_setup(args, use_graphs: bool):
    """A model of the layer sizes that --shape names whose cache holds random keys and values, and a
    function that runs decode step i."""
    import numpy as np

    from ..engine import Engine
    cfg = _config(args)
    B, C = args.batch, args.context
    longest = 2 * C if args.unequal else C
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=B * (longest + 64), max_batch=B,
                             max_context=longest + 64, use_graphs=use_graphs)
    for g in eng.cache.kv_groups:
        g.k_pages.normal_()
        g.v_pages.normal_()
    slots = [eng.new_sequence() for _ in range(B)]
    start = C - args.iters - args.warmup
    for i, s in enumerate(slots):         # the cache holds `start` tokens of random keys and values
        # --unequal: lengths from a twentieth of the context to almost twice it, the same mean
        n = start if not args.unequal or B == 1 else max(1, int(start * (0.05 + 1.9 * i / (B - 1))))
        eng.cache.reserve(s, n)
        eng.cache.commit(s, n)
    rng = np.random.default_rng(0)
    feed = rng.integers(0, cfg["vocab_size"], (args.iters + args.warmup, B))

    def run(i):
        eng.step([(s, [int(t)]) for s, t in zip(slots, feed[i])])
    return run


def bench_step(args) -> dict:
    B, C = args.batch, args.context
    run = _decode_setup(args, not args.eager)
    ms = _time(run, args.iters, args.warmup, graph=False)
    return {"kernel": "decode step", "batch": B, "context": C, "layers": args.layers, "graph": not args.eager,
            "ms": ms, "tokens_per_s": B / ms * 1e3}


def bench_timeline(args) -> dict:
    """Kernel records of the last of `--iters` decode steps: per kind of kernel the launches, the
    mean run time, and the mean time by which it ended after the kernel before it."""
    import re

    from torch.profiler import ProfilerActivity, profile
    run = _prefill_setup(args) if args.prompt else _decode_setup(args, True)
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(args.iters):
            run(args.warmup + i)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and not re.search("[Mm]emcpy|[Mm]emset", e.name)]
    ev.sort(key=lambda e: e.time_range.start)
    starts = [i for i, e in enumerate(ev) if e.name == ev[0].name]          # the step's first kernel runs once a step
    last = ev[starts[-2]:starts[-1]] if len(starts) >= 2 else ev

    def kind(name: str) -> str:
        m = re.search(r"(\w+)_kernel<([^>]*)>", name)
        return f"{m.group(1)}<{m.group(2)[:40]}>" if m else name[:60]
    t0 = prev_end = last[0].time_range.start
    kinds: dict = {}
    for e in last:
        k = kinds.setdefault(kind(e.name), dict(launches=0, run_us=0.0, adds_us=0.0))
        k["launches"] += 1
        k["run_us"] += e.time_range.end - e.time_range.start
        k["adds_us"] += e.time_range.end - prev_end if e is not last[0] else e.time_range.end - t0
        prev_end = max(prev_end, e.time_range.end)
    for k in kinds.values():
        k["run_us"] = round(k["run_us"] / k["launches"], 2)
        k["adds_us"] = round(k["adds_us"] / k["launches"], 2)
    return {"kernel": ("prompt" if args.prompt else "decode") + " step, kernel by kernel", "shape": args.shape, "batch": args.batch, "context": args.context, "layers": args.layers,
            "step_us": round(prev_end - t0, 1), "kinds": kinds}


def _prefill_setup(args):
    """A model of the layer sizes that --shape names and a function that runs a prompt of --tokens tokens."""
    import numpy as np

    from ..engine import Engine
    cfg = _config(args)
    T = args.tokens
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=T + 64, max_batch=1, max_context=T + 64)
    rng = np.random.default_rng(0)

    def run(i):
        slot = eng.new_sequence()
        eng.step([(slot, rng.integers(0, cfg["vocab_size"], T).tolist())])
        eng.end_sequence(slot)
    return run


def bench_prefill(args) -> dict:
    T = args.tokens
    run = _prefill_setup(args)
    ms = _time(run, args.iters, args.warmup, graph=False)
    return {"kernel": "prefill step", "tokens": T, "layers": args.layers, "ms": ms, "tokens_per_s": T / ms * 1e3}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=["gemm_skinny", "gemm_tc", "attn_decode", "attn_prefill", "attn_prefill_tc", "chain", "step",
                                     "prefill", "timeline", "sample"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--epi", default="bf16", choices=sorted(EPIS))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes for step, timeline and prefill")
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--one-block", action="store_true", help="sample: the kernel that takes a row per block")
    ap.add_argument("--unequal", action="store_true",
                    help="step, timeline: sequences of unequal lengths (a twentieth to twice --context, the same mean)")
    ap.add_argument("--equal-slices", action="store_true",
                    help="step, timeline: decode attention cuts every sequence into the same number of slices "
                         "instead of giving every team of blocks an equal share of all keys")
    ap.add_argument("--single-sm", action="store_true",
                    help="gemm_tc, prefill: every tile on one SM (no products on pairs of SMs)")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--prompt", action="store_true", help="timeline: a prompt step of --tokens tokens instead of a decode step")
    ap.add_argument("--no-graph", action="store_true", help="time single kernels launch by launch from the host")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    global GRAPH
    GRAPH = not args.no_graph
    if args.single_sm:
        from . import ops
        ops.USE_PAIRS = False
    if args.equal_slices:
        from . import attention
        attention.BALANCED_DECODE = False
    if args.what in ("gemm_skinny", "gemm_tc"):
        out = bench_gemm(args.what, args)
    elif args.what == "chain":
        out = bench_chain(args)
    elif args.what == "sample":
        out = bench_sample(args)
    elif args.what == "attn_decode":
        out = bench_attn_decode(args)
    elif args.what in ("attn_prefill", "attn_prefill_tc"):
        out = bench_attn_prefill(args)
    elif args.what == "prefill":
        out = bench_prefill(args)
    elif args.what == "timeline":
        out = bench_timeline(args)
    else:
        out = bench_step(args)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
