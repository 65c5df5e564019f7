"""Plain, slow Llama 3 decoder: the oracle that every engine test compares with.

Whole sequences, no cache, no batching, one function for each part, float64 by
default.  It shares no code with the product: it reads config.json as a plain
dict, reads safetensors with its own few lines, and computes every formula the
way the reference's engine does, cited by file:line of 23skdu/longbow-quarrel.

This file rests on the reference's formulas only: the reference is a Go program
whose one complete forward pass runs on Apple Metal, and neither a Go toolchain
nor Metal exists where these tests run, so its model code cannot be imported or
compiled to make golden outputs.  The Llama 3 `rope_scaling` rule is not in the
reference at all (its RoPE is the unscaled `theta^(-2i/d)` of
internal/device/kernels.metal:452); it is restated here from the public
description of the "llama3" rope type that config.json files carry.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, a JSON header, raw tensor bytes."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo:8 + n + hi])
        t = torch.frombuffer(buf, dtype=_ST_DTYPES[info["dtype"]]) if hi > lo else \
            torch.empty(0, dtype=_ST_DTYPES[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return cfg, weights


# --------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """Row `tok` of the table, no multiplier: internal/device/kernels.metal:465-467
    (embedding_f16); the range check is internal/engine/engine.go:1327-1331."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    assert int(tokens.min()) >= 0 and int(tokens.max()) < table.shape[0]
    return table[tokens]


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i * 1/sqrt(mean(x^2) + eps) * w_i, eps inside the root and added to
    the mean, no +1 on the gain: internal/device/kernels.metal:916-940
    (rmsnorm_f32_to_f16_v4); internal/device/cpu_ref.go:62-82 (CPURMSNorm)."""
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return x * scale * gain


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x . W^T with W stored [out, in], no bias: internal/device/cpu_ref.go:85-97
    (CPUMatMul, "B is transposed"); internal/device/kernels.metal:115-131 (linear_f16)."""
    return x @ w.T


def rope_frequencies(head_dim: int, theta: float, scaling: dict | None) -> np.ndarray:
    """f_i = theta^(-2i/head_dim) for i < head_dim/2: internal/device/kernels.metal:452,
    internal/device/cpu_ref.go:117.  With rope_scaling of type "llama3" (not in the
    reference) a frequency whose wavelength is longer than n0/low is divided by
    `factor`, one shorter than n0/high is kept, and the band between is blended."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    f = theta ** (-2.0 * i / head_dim)
    if not scaling:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return f
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    n0 = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(f)
    for j, fj in enumerate(f):
        wavelen = 2.0 * math.pi / fj
        if wavelen < n0 / hi:
            out[j] = fj
        elif wavelen > n0 / lo:
            out[j] = fj / factor
        else:
            s = (n0 / wavelen - lo) / (hi - lo)
            out[j] = (1.0 - s) * fj / factor + s * fj
    return out


def rope(x: torch.Tensor, positions, freqs: np.ndarray) -> torch.Tensor:
    """Half-split rotation: element i pairs with i + head_dim/2;
    x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos, angle = position * f_i:
    internal/device/kernels.metal:443-461 (rope_f16), internal/device/cpu_ref.go:100-131.
    x is [T, heads, head_dim]."""
    half = x.shape[-1] // 2
    ang = torch.as_tensor(np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :])
    cos, sin = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention(q, k, v, scale: float, window: int | None = None, round_probabilities=None) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.
    kv head of query head h is h // (H / Hkv): internal/device/kernels.metal:671;
    score = q.k * scale over keys start..p, own position included (:697-704);
    start = p - window + 1 when a window is set and p >= window (:676);
    softmax with the maximum subtracted (:710-756); out = sum_t p_t v_t (:759-766).
    q [T, H, hd], k and v [T, Hkv, hd] -> [T, H, hd].
    round_probabilities: a function applied to exp(s - max) before the sum and the product with v (see
    `forward(storage=...)`)."""
    T, H, hd = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    out = torch.empty_like(q)
    idx = torch.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window:
        allowed &= idx[None, :] > (idx[:, None] - window)
    for h in range(H):
        kvh = h // group
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        if round_probabilities is None:
            p = torch.softmax(s, dim=-1)
        else:
            e = round_probabilities(torch.exp(s - s.max(dim=-1, keepdim=True).values))
            p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """up * silu(gate), silu(g) = g / (1 + e^-g), no clamp:
    internal/device/cpu_ref.go:133-149 (CPUSwiGLU); internal/device/cuda_kernels.cu:28-37."""
    return up * (gate / (1.0 + torch.exp(-gate)))


# --------------------------------------------------------------------------- model

def _cfg(cfg: dict):
    D = cfg["hidden_size"]
    H = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or D // H
    return D, H, Hkv, hd


def layer_window(cfg: dict, layer: int) -> int | None:
    """The window of a layer: `sliding_window` where `layer_types` says
    "sliding_attention" (every layer when there is a window but no list)."""
    w = cfg.get("sliding_window")
    if not w:
        return None
    types = cfg.get("layer_types")
    if types is None or types[layer] == "sliding_attention":
        return int(w)
    return None


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, start_pos: int = 0,
            return_hidden: bool = False, return_layers: bool = False, storage=None):
    """Logits [T, vocab] at every position of one whole sequence (with return_layers: also the residual
    stream after the embedding and after every layer, both as numpy arrays).
    Block order x += Attn(norm(x)); x += FFN(norm(x)) with two pre-norms:
    internal/device/metal.go:1347-1527 (Tensor.Layer); final norm and LM head:
    internal/engine/engine.go:1547,1561; tied head when there is no lm_head tensor:
    internal/engine/engine.go:1108-1111.

    storage: a dtype (torch.bfloat16) in which activations are kept between the operations, as an engine
    of that precision keeps them: the normed rows, q, k and v, the probabilities, the attention's output
    and the feed-forward's inner rows are rounded to it; sums, norms, softmax and the residual stream stay
    in `dtype`.  The difference to the unrounded result is the error that this storage precision alone
    causes, whatever the kernels: the yardstick for what an engine of that precision may differ by."""
    D, H, Hkv, hd = _cfg(cfg)
    keep = (lambda t: t) if storage is None else (lambda t: t.to(storage).to(dtype))
    eps = cfg.get("rms_norm_eps", 1e-5)
    freqs = rope_frequencies(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    W = {k: v.to(dtype) for k, v in weights.items()}
    T = len(tokens)
    pos = np.arange(start_pos, start_pos + T)
    x = embedding(W["model.embed_tokens.weight"], tokens)
    layers = [x.numpy().copy()]            # the residual stream after the embedding and after every layer
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = keep(rms_norm(x, W[p + "input_layernorm.weight"], eps))
        q = linear(n, W[p + "self_attn.q_proj.weight"]).reshape(T, H, hd)
        k = linear(n, W[p + "self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
        v = keep(linear(n, W[p + "self_attn.v_proj.weight"]).reshape(T, Hkv, hd))
        q, k = keep(rope(q, pos, freqs)), keep(rope(k, pos, freqs))
        a = keep(attention(q, k, v, hd ** -0.5, layer_window(cfg, l),
                           None if storage is None else keep).reshape(T, H * hd))
        x = x + linear(a, W[p + "self_attn.o_proj.weight"])
        n = keep(rms_norm(x, W[p + "post_attention_layernorm.weight"], eps))
        g = linear(n, W[p + "mlp.gate_proj.weight"])
        u = linear(n, W[p + "mlp.up_proj.weight"])
        x = x + linear(keep(swiglu(g, u)), W[p + "mlp.down_proj.weight"])
        layers.append(x.numpy().copy())
    if return_hidden:
        return x
    n = keep(rms_norm(x, W["model.norm.weight"], eps))
    head = W["lm_head.weight"] if "lm_head.weight" in W else W["model.embed_tokens.weight"]
    if return_layers:
        return linear(n, head).numpy(), np.stack(layers)       # logits [T, vocab], stream [layers + 1, T, D]
    return linear(n, head)


def greedy(cfg: dict, weights: dict, prompt, n_new: int, stop=()) -> list[int]:
    """Greedy generation by re-running the whole sequence for each token
    (as cmd/debug_generation/main.go:61-93 does); first maximum wins
    (internal/engine/sampler.go:282-307); a stop token ends the sequence and is
    not returned (internal/engine/engine.go:1744)."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        logits = forward(cfg, weights, seq)[-1]
        tok = int(torch.argmax(logits))
        if tok in stop:
            break
        out.append(tok)
        seq.append(tok)
    return out


# --------------------------------------------------------------------------- sampling

def kept_set(logits, temperature, top_k, top_p):
    """The tokens the reference sampler keeps, and their probabilities:
    softmax(logits / T) in float64; drop p <= 1e-10; sort by falling probability; keep
    the first k; keep the shortest prefix whose sum reaches top_p and renormalise:
    internal/engine/sampler.go:125-166,309-339.  Ties are ordered by index here (the
    reference's sort leaves their order open).  Returned in index order."""
    logits = np.asarray(logits, dtype=np.float64)
    z = logits / temperature
    p = np.exp(z - z.max())
    p /= p.sum()
    ids = [i for i in range(len(p)) if p[i] > 1e-10]
    ids.sort(key=lambda i: (-p[i], i))
    if 0 < top_k < len(ids):
        ids = ids[:top_k]
    probs = np.array([p[i] for i in ids])
    if 0.0 < top_p < 1.0:
        c = np.cumsum(probs)
        if c[-1] >= top_p:
            n = int(np.searchsorted(c, top_p, side="left")) + 1
            ids, probs = ids[:n], probs[:n] / probs[:n].sum()
    order = np.argsort(ids)
    return [int(ids[i]) for i in order], [float(probs[i]) for i in order]


def sample_reference(logits, temperature, top_k, top_p, u: float) -> int:
    """The decision for one uniform draw u in [0, 1): greedy at temperature 0
    (internal/engine/sampler.go:81-84); else r = u * sum of the kept probabilities and a
    walk along their cumulative sum until r < acc (sampler.go:168-184).  The reference
    walks in sorted order; the walk here is in index order, which draws from the same
    distribution."""
    if temperature == 0:
        return int(np.argmax(np.asarray(logits, dtype=np.float64)))
    ids, probs = kept_set(logits, temperature, top_k, top_p)
    r = u * sum(probs)
    acc = 0.0
    for i, pi in zip(ids, probs):
        acc += pi
        if r < acc:
            return int(i)
    return int(ids[-1])


def philox_uniform(seed: int, sequence: int, step: int) -> float:
    """Philox4x32-10 with key = seed and counter = (sequence, step, 0, 0); the first two
    output words give a 53-bit uniform number in [0, 1) (public algorithm of Salmon et al.,
    "Parallel random numbers: as easy as 1, 2, 3")."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [sequence & 0xFFFFFFFF, step & 0xFFFFFFFF, 0, 0]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k0, p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k1, p0 & 0xFFFFFFFF]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return (((c[0] >> 5) << 26) | (c[1] >> 6)) / float(1 << 53)


def repetition_penalty(logits, history, penalty: float):
    """Unique ids among the last 64 history tokens: a positive logit is divided by
    the penalty, a negative one multiplied: internal/engine/sampler.go:249-275."""
    out = np.array(logits, dtype=np.float64)
    if penalty <= 1.0:
        return out
    for t in set(history[-64:]):
        if t < len(out):
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out
