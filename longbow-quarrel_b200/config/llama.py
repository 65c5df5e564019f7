"""Typed configuration of the Llama 3 dense decoder, read from its config.json keys.

The reference fills a `config.Config` from GGUF metadata with the same meanings
(internal/engine/engine.go:452-588: block_count, embedding_length,
attention.head_count, head_count_kv, feed_forward_length, rope.freq_base,
layer_norm_rms_epsilon, context_length) and validates it in
internal/config/config.go:57-105.  Here the keys are those of config.json.
`head_dim` is a key of its own (the reference fixes it to hidden/heads,
internal/engine/engine.go:509-511), `rope_scaling` of type "llama3" is read (the
reference has no scaling rule), and an optional `sliding_window` with
`layer_types` gives single layers the window of the reference's attention kernel
(internal/device/kernels.metal:676).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field

from .base import ConfigError, KeyReader, read_config_json

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of type "llama3": wavelengths longer than
    original_max_position_embeddings / low_freq_factor are stretched by `factor`,
    those shorter than original / high_freq_factor are kept, the band between is
    blended linearly."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, data: dict | None) -> "RopeScaling | None":
        if data is None:
            return None
        if not isinstance(data, dict):
            raise ConfigError(f"config.json: 'rope_scaling' must be an object or null, found {data!r}")
        r = KeyReader(data, "config.json: rope_scaling")
        kind = data.get("rope_type", data.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (supported: 'llama3', 'default')")
        out = cls(rope_type="llama3",
                  factor=r.number("factor", positive=True),
                  low_freq_factor=r.number("low_freq_factor", positive=True),
                  high_freq_factor=r.number("high_freq_factor", positive=True),
                  original_max_position_embeddings=r.integer("original_max_position_embeddings", minimum=1))
        if not out.high_freq_factor > out.low_freq_factor:
            raise ConfigError("config.json: rope_scaling.high_freq_factor must be greater than low_freq_factor")
        return out


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: tuple[int, ...] = ()
    sliding_window: int | None = None
    layer_types: tuple[str, ...] | None = None
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = field(default=("LlamaForCausalLM",))

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: dict) -> "LlamaConfig":
        r = KeyReader(data)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        for key in ("attention_bias", "mlp_bias"):
            if r.boolean(key, False):
                raise ConfigError(f"config.json: '{key}': true is not supported (the architecture has no biases)")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', found {act!r}")
        head_dim = r.integer("head_dim", None, minimum=1)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads
        layer_types = data.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or not all(isinstance(t, str) for t in layer_types):
                raise ConfigError("config.json: 'layer_types' must be a list of strings")
            layer_types = tuple(layer_types)
        bos = r.integer("bos_token_id", None)
        archs = data.get("architectures") or ["LlamaForCausalLM"]
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            num_key_value_heads=r.integer("num_key_value_heads", heads, minimum=1),
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps", 1e-5, positive=True),
            rope_theta=r.number("rope_theta", 10000.0, positive=True),
            rope_scaling=RopeScaling.from_dict(data.get("rope_scaling")),
            max_position_embeddings=r.integer("max_position_embeddings", 2048, minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            bos_token_id=bos,
            eos_token_id=r.int_or_list("eos_token_id"),
            sliding_window=r.integer("sliding_window", None, minimum=1),
            layer_types=layer_types,
            torch_dtype=r.string("torch_dtype", data.get("dtype") or "bfloat16"),
            architectures=tuple(archs),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, folder_or_file) -> "LlamaConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        """The checks of internal/config/config.go:57-105, less `dim == heads *
        head_dim` (head_dim is free here), plus heads % kv_heads == 0, which the
        reference checks only when attention runs (internal/device/metal.go:1757-1761)."""
        if self.num_key_value_heads > self.num_attention_heads:
            raise ConfigError(f"config.json: num_key_value_heads {self.num_key_value_heads} exceeds "
                              f"num_attention_heads {self.num_attention_heads}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotary pairs)")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"config.json: layer_types has {len(self.layer_types)} entries for "
                                  f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                    raise ConfigError(f"config.json: layer type {t!r} is not one of "
                                      f"'{FULL_ATTENTION}', '{SLIDING_ATTENTION}'")
            if SLIDING_ATTENTION in self.layer_types and not self.sliding_window:
                raise ConfigError("config.json: layer_types names sliding_attention but 'sliding_window' is not set")

    # ------------------------------------------------------------------ derived
    def window_of_layer(self, layer: int) -> int | None:
        if not self.sliding_window:
            return None
        if self.layer_types is None or self.layer_types[layer] == SLIDING_ATTENTION:
            return self.sliding_window
        return None

    def to_dict(self) -> dict:
        out = asdict(self)
        out["architectures"] = list(self.architectures)
        out["model_type"] = "llama"
        out["hidden_act"] = "silu"
        out["attention_bias"] = False
        out["mlp_bias"] = False
        eos = self.eos_token_id
        out["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        if self.layer_types is not None:
            out["layer_types"] = list(self.layer_types)
        return out
