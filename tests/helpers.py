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
}


def make_model_folder(tmp: Path, name: str, seed: int = 0, dtype=torch.bfloat16, gain_std: float = 0.1,
                      std: float = 0.02, overrides: dict | None = None) -> Path:
    """A model folder with random weights, written by the framework's random-weights mode."""
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    from longbow_quarrel_b200.engine.model import Model
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.weights import write_random_model
    from longbow_quarrel_b200 import architectures  # noqa: F401
    cfg_dict = {**TINY[name], **(overrides or {})}
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


# What each precision must reach against the float64 plain implementation.
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
