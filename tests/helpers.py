"""Tiny configurations, model folders with random weights, and the error measures
that the engine tests share."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import plain_llama

# Three tiny configurations of the architecture that differ in every size and option.
TINY = {
    # 2:1 groups, head_dim 16, an intermediate size that is no multiple of 64, untied head
    "A": dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
              rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=128,
              eos_token_id=255),
    # one kv head for three heads, head_dim 32, llama3 rope scaling that hits all three branches, tied head
    "B": dict(architectures=["LlamaForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=384, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256, eos_token_id=[7, 9]),
    # heads * head_dim != hidden, as many kv heads as heads, a vocabulary that is no multiple of 8,
    # a window on every other layer
    "C": dict(architectures=["LlamaForCausalLM"], hidden_size=80, num_hidden_layers=4, num_attention_heads=5,
              num_key_value_heads=5, head_dim=48, intermediate_size=200, vocab_size=250, rope_theta=1000000.0,
              rope_scaling=None, rms_norm_eps=3e-5, tie_word_embeddings=True, max_position_embeddings=512,
              sliding_window=40, layer_types=["sliding_attention", "full_attention"] * 2, eos_token_id=None),
    # the sizes that take the tensor-core kernels of real models, small: head_dim 64, one kv head for two heads,
    # a window of 100 on every other layer, room for prompts of several hundred tokens
    "D": dict(architectures=["LlamaForCausalLM"], hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
              num_key_value_heads=1, head_dim=64, intermediate_size=320, vocab_size=500, rope_theta=10000.0,
              rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024,
              sliding_window=100, layer_types=["sliding_attention", "full_attention"], eos_token_id=None),
    # head_dim 128 with heads * head_dim != hidden, one layer
    "E": dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=1, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=777, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=256),
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024, eos_token_id=None),
}

# Layers of the sizes that real checkpoints have (two of them), with the vocabulary cut so that the plain
# implementation still runs in seconds on the CPU.
REAL = {
    "8B": dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=2, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=4000, rope_theta=500000.0,
               rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192),
               rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=4096, eos_token_id=None),
    "1B": dict(architectures=["LlamaForCausalLM"], hidden_size=2048, num_hidden_layers=2, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=3000, rope_theta=500000.0,
               rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192),
               rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=4096, eos_token_id=None),
}


def make_model_folder(tmp: Path, name, seed: int = 0, dtype=torch.bfloat16, gain_std: float = 0.1,
                      std: float = 0.02, overrides: dict | None = None) -> Path:
    """A model folder with random weights, written by the framework's random-weights mode."""
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    from longbow_quarrel_b200.engine.model import Model
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.weights import write_random_model
    from longbow_quarrel_b200 import architectures  # noqa: F401
    base = name if isinstance(name, dict) else TINY[name] if name in TINY else REAL[name]
    cfg_dict = {**base, **(overrides or {})}
    name = name if isinstance(name, str) else "custom"
    arch = architecture_of(cfg_dict)
    cfg = arch.config_from_dict(cfg_dict)
    model = Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, cfg.max_position_embeddings))
    folder = Path(tmp) / f"tiny_{name}_{seed}"
    return write_random_model(folder, cfg.to_dict(), model.weight_table(), seed, dtype, std, gain_std)


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def plain_logits(folder: Path, tokens: list[int]) -> np.ndarray:
    cfg, weights = plain_llama.load_folder(folder)
    return plain_llama.forward(cfg, weights, tokens).numpy()


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Largest difference over the root mean square of the reference."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite values"
    return float(np.abs(got - ref).max() / max(np.sqrt((ref * ref).mean()), 1e-30))


def rel_l2(got: np.ndarray, ref: np.ndarray) -> float:
    """Root mean square of the difference over the root mean square of the reference: unlike the largest
    difference it does not grow with the number of values looked at."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite values"
    return float(np.sqrt(((got - ref) ** 2).mean()) / max(np.sqrt((ref * ref).mean()), 1e-30))


class Errors:
    """Collects the worst error of every kind of comparison, so that a test can print them all and then
    judge them: a failure shows the whole picture, not the first number over its bound."""

    def __init__(self):
        self.worst: dict[str, tuple[float, object]] = {}

    def add(self, kind: str, err: float, where=None) -> None:
        if kind not in self.worst or err > self.worst[kind][0]:
            self.worst[kind] = (err, where)

    def __str__(self):
        return ", ".join(f"{k} {v:.3g}" + (f" at {w}" if k.startswith("same") else "") for k, (v, w) in self.worst.items())

    def check(self, bounds: dict[str, float]) -> None:
        """bounds: prefix of kind -> bound (the longest matching prefix counts; every kind must match one)."""
        bad = []
        for kind, (err, where) in self.worst.items():
            match = max((p for p in bounds if kind.startswith(p)), key=len, default=None)
            assert match is not None, f"no bound for {kind}"
            if not err < bounds[match]:
                bad.append(f"{kind}: {err:.3g} is not below {bounds[match]:.3g} (at {where})")
        assert not bad, "; ".join(bad) + f" -- all: {self}"


def storage_noise(cfg: dict, weights: dict, tokens: list[int], exact: np.ndarray | None = None) -> tuple[float, float]:
    """The yardstick for a bfloat16 engine on this request: how far the plain implementation itself moves
    when it keeps its activations in bfloat16 between the operations (everything else in float64), as
    (worst rel_l2, worst rel_err) over the positions.  An engine that stores activations in bfloat16 cannot
    be closer to the exact result than this, whatever its kernels; and because a difference far below one
    rounding step becomes a whole step wherever it tips a rounding, two correct bfloat16 paths that sum
    in another order end up this far from each other, too, after a few operations."""
    import torch
    if exact is None:
        exact = plain_llama.forward(cfg, weights, tokens).numpy()
    stored = plain_llama.forward(cfg, weights, tokens, storage=torch.bfloat16).numpy()
    n = len(tokens)
    return max(rel_l2(stored[i], exact[i]) for i in range(n)), max(rel_err(stored[i], exact[i]) for i in range(n))


def bounds(dtype: str, noise: tuple[float, float] | None = None) -> dict[str, float]:
    """Bounds for `Errors.check` by kind of comparison.  float32: the plain implementation to 1e-4 and two
    cuts of the same request to 2e-5 of the logits' root mean square (in practice they are equal bit by
    bit).  bfloat16: one and a half times the storage noise of the request set (`storage_noise`), for the root mean
    square of a row's difference ("l2") and for its largest entry ("max").  Measured on B200, the engine's
    distance to the exact result is 1.0 to 1.1 times that noise at every size tried (two layers of the 1B and
    8B shapes, tiny models with weights five times larger), and two cuts lie 0.5 to 0.9 times it apart."""
    if dtype == "float32":
        return {"plain": TOL["float32"], "same": 2e-5, "other": 2e-5}
    l2, worst = noise
    return {"plain l2": 1.5 * l2, "plain max": 1.5 * worst, "same l2": 1.5 * l2, "same max": 1.5 * worst,
            "other l2": 1.5 * l2, "other max": 1.5 * worst}


_tolerances: dict = {}


def tolerance(dtype: str, folder, tokens) -> float:
    """The bound on a row's largest difference from the plain implementation, over the root mean square of the
    row: 1e-4 in float32; in bfloat16 one and a half times what keeping the activations in bfloat16 costs the
    plain implementation itself on this request (`storage_noise`), so a model whose weights make rounding
    matter little (small tiny models: about 1 %) is held to that, not to a bound that fits every model."""
    if dtype == "float32":
        return TOL["float32"]
    key = (str(folder), tuple(tokens))
    if key not in _tolerances:
        cfg, weights = plain_llama.load_folder(folder)
        _tolerances[key] = 1.5 * storage_noise(cfg, weights, list(tokens))[1]
    return _tolerances[key]


def assert_rows_close(got: np.ndarray, ref: np.ndarray, tol: float, what="") -> float:
    """Every row of got within tol of its row of ref (rel_err); returns the worst."""
    worst = 0.0
    for i in range(len(ref)):
        err = rel_err(got[i], ref[i])
        assert err < tol, f"{what} row {i} of {len(ref)}: error {err:.3g} is not below {tol:.3g}"
        worst = max(worst, err)
    return worst


# What each precision must reach against the float64 plain implementation.
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
