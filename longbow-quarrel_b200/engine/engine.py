"""The Python entry point: a model with its cache on one GPU.

It mirrors the reference's Engine interface -- Infer / InferWithCallback / Close
(internal/engine/types_base.go:17-21) with a SamplerConfig (types_base.go:7-15) --
as generate() with SamplingParams, and adds what the reference lacks: batches of
sequences, and the step function that both generation and trace replay drive.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .. import architectures  # noqa: F401  (registers the architectures)
from ..cache import Cache
from ..config.registry import architecture_of, load_config
from ..kernels import ops
from ..parts.base import Runtime
from ..weights import load_weights, random_weights
from .model import Model
from ..sampling import SamplingParams
from .generate import GenerationStats, generate
from .step import Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', found {name!r}") from None


def _device(device) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("longbow-quarrel_b200 runs on a CUDA GPU (sm_100a); none is visible. "
                           "There is no CPU path.")
    return torch.device(device)


class Engine:
    def __init__(self, arch, config, model: Model, cache: Cache, runtime: Runtime, use_graphs: bool = True):
        self.arch, self.config, self.model, self.cache, self.runtime = arch, config, model, cache, runtime
        self.device = runtime.device
        self.stepper = Stepper(model, cache, self.device, use_graphs=use_graphs)
        self.last_stats: GenerationStats | None = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def _build(cls, arch, config, tensors_fn, dtype, max_tokens, max_batch, max_context, device, use_graphs=True):
        dtype, device = _dtype(dtype), _device(device)
        spec = arch.describe(config)
        max_context = min(max_context or spec.max_positions, spec.max_positions)
        max_tokens = max_tokens or max_context
        max_context = min(max_context, -(-max_tokens // 64) * 64)
        runtime = Runtime(device=device, dtype=dtype, max_context=max_context)
        ops.prepare(dtype)
        with torch.cuda.device(device):
            model = Model(spec, runtime)
            tensors = tensors_fn(model.weight_table(), device)
            model.load(tensors)
            del tensors
            cache = Cache(model.cache_needs(), max_tokens, max_context, dtype, device, max_slots=max_batch)
        return cls(arch, config, model, cache, runtime, use_graphs)

    @classmethod
    def from_pretrained(cls, folder, dtype="bfloat16", max_tokens: int | None = None, max_batch: int | None = None,
                        max_context: int | None = None, device="cuda:0", use_graphs: bool = True,
                        convert_weights: bool = False, unexpected: str = "error") -> "Engine":
        """A model folder (config.json + model.safetensors); the class is chosen by config.json.

        Weights are kept as the file stores them.  A tensor stored in 32-bit therefore stays so under
        dtype="bfloat16" too, and its products run on the CUDA cores instead of the tensor cores: right,
        but several times slower, so a warning says it.  convert_weights=True rounds the weights to the
        model's precision as they are loaded instead (what the reference does,
        internal/engine/engine.go:787-802).  unexpected: see weights.load_weights."""
        folder = Path(folder)
        arch, config = load_config(folder)
        run_dtype = _dtype(dtype)

        def tensors(table, dev):
            out = load_weights(folder, table, dev, convert_to=run_dtype if convert_weights else None, unexpected=unexpected)
            wide = [n for n, t in out.items() if t.dtype == torch.float32 and t.dim() >= 2]
            if wide and run_dtype == torch.bfloat16:
                import warnings
                warnings.warn(f"{folder}: {len(wide)} weight matrices are stored in 32-bit; with dtype='bfloat16' their "
                              f"products run on the CUDA cores (pass convert_weights=True to round them to bfloat16 at load)")
            return out
        return cls._build(arch, config, tensors, dtype, max_tokens, max_batch, max_context, device, use_graphs)

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype="bfloat16", max_tokens: int | None = None,
                    max_batch: int | None = None, max_context: int | None = None, device="cuda:0",
                    std: float = 0.02, gain_std: float = 0.0, weight_dtype=torch.bfloat16,
                    use_graphs: bool = True) -> "Engine":
        """Random weights made on the device (a dict with config.json's keys, or a typed config)."""
        if isinstance(config, dict):
            arch = architecture_of(config)
            config = arch.config_from_dict(config)
        else:
            arch = architecture_of({"architectures": list(config.architectures)})
        return cls._build(arch, config,
                          lambda table, dev: random_weights(table, seed, weight_dtype, dev, std, gain_std),
                          dtype, max_tokens, max_batch, max_context, device, use_graphs)

    # ------------------------------------------------------------------ sequences and steps
    def new_sequence(self) -> int:
        """A slot for a sequence that starts now."""
        return self.cache.alloc_slot()

    def end_sequence(self, slot: int) -> None:
        """Give back what the sequence holds."""
        self.cache.free_slot(slot)

    def step(self, entries, want=None) -> torch.Tensor | None:
        """Run the next tokens of each sequence: entries = [(slot, tokens)], either whole
        prompts or one token each; want = for each entry the places among its tokens whose
        logits are asked for (None: each entry's last).  Returns float32 [n_wanted, vocab]."""
        with torch.cuda.device(self.device):
            return self.stepper.step(entries, want)

    def check(self) -> None:
        """Raise if a kernel of an earlier step gave up a bounded wait (its results are then not valid).  Sees
        the steps that the host has waited for: call it after reading a step's logits."""
        ops.check_status()

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, max_new_tokens: int = 20, sampling: SamplingParams | None = None, stop_ids=None,
                 callback=None, include_stop: bool = False, batch_size: int | None = None,
                 logits_callback=None) -> list[list[int]]:
        """New tokens for each prompt (lists of token ids).  Prompts are run in batches of
        at most batch_size that start together; a sequence ends at a stop token (by default
        the model's eos ids; the stop token is not returned), after max_new_tokens, or when
        the context is full.  callback(prompt index, token id) is called for every token;
        logits_callback(prompt index, step, logits) with the float32 logits (on the host) from which the
        token of that step was sampled, before the token's own callback (it costs a copy of every step's
        logits and the overlap of steps with the host's work).
        Counterpart of Infer / InferWithCallback / InferWithCallbackLogits (internal/engine/engine.go:1277-1290)."""
        from .backend import EngineBackend
        sampling = sampling or SamplingParams()
        stops = tuple(self.model.spec.stop_tokens) if stop_ids is None else tuple(stop_ids)
        with torch.cuda.device(self.device):
            outputs, stats = generate(EngineBackend(self, sampling, logits_callback=logits_callback), prompts, max_new_tokens, stops, callback,
                                      include_stop, batch_size or self.cache.max_slots,
                                      self.runtime.max_context)
        self.last_stats = stats
        return outputs

    def close(self) -> None:
        self.model = None
        self.cache = None
