"""Configuration: reading config.json keys, defaults, errors that name the key, the registry."""
import json

import pytest

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200 import architectures  # noqa: F401
from longbow_quarrel_b200.config import (ConfigError, LlamaConfig, RopeScaling, architecture_of, load_config,
                                         register_architecture, registered_architectures)
from helpers import TINY


def test_reads_every_key():
    cfg = LlamaConfig.from_dict(TINY["B"])
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (96, 3, 3, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 256, 384)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0
    assert cfg.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    assert cfg.tie_word_embeddings is True and cfg.max_position_embeddings == 256
    assert cfg.eos_token_id == (7, 9)


def test_defaults_follow_the_reference():
    cfg = LlamaConfig.from_dict(dict(hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
                                     intermediate_size=128, vocab_size=100))
    assert cfg.num_key_value_heads == 4          # kv heads default to heads
    assert cfg.head_dim == 16                    # hidden / heads
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.max_position_embeddings == 2048
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False and cfg.eos_token_id == ()
    assert cfg.sliding_window is None and cfg.window_of_layer(0) is None


def test_head_dim_is_free():
    cfg = LlamaConfig.from_dict(TINY["C"])
    assert cfg.num_attention_heads * cfg.head_dim != cfg.hidden_size
    assert [cfg.window_of_layer(i) for i in range(4)] == [40, None, 40, None]


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size"])
def test_missing_required_key_is_named(key):
    data = dict(TINY["A"])
    del data[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(data)


@pytest.mark.parametrize("patch,match", [
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"num_key_value_heads": 8}, "exceeds"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 4.0, "high_freq_factor": 1.0,
                       "original_max_position_embeddings": 64}}, "high_freq_factor"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"tie_word_embeddings": 1}, "tie_word_embeddings"),
])
def test_bad_values_are_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict({**TINY["A"], **patch})


def test_rope_scaling_default_type_means_none():
    cfg = LlamaConfig.from_dict({**TINY["A"], "rope_scaling": {"rope_type": "default"}})
    assert cfg.rope_scaling is None


def test_round_trip_through_json(tmp_path):
    cfg = LlamaConfig.from_dict(TINY["C"])
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    arch, again = load_config(tmp_path)
    assert arch.name == "LlamaForCausalLM" and again == cfg


def test_registry_names_unknown_architecture(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="NoSuchModel.*LlamaForCausalLM"):
        architecture_of({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({})
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(tmp_path)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path / "nowhere")


def test_registering_another_architecture():
    register_architecture("ToyForTest", lambda d: d, lambda c: None)
    assert architecture_of({"architectures": ["ToyForTest"]}).name == "ToyForTest"


def test_describe_takes_every_constant_from_the_config():
    from longbow_quarrel_b200.architectures.llama import describe
    for name in TINY:
        cfg = LlamaConfig.from_dict(TINY[name])
        spec = describe(cfg)
        assert len(spec.layers) == cfg.num_hidden_layers == len(spec.schedule)
        mixer = spec.layers[0].part("mixer").params
        assert mixer["n_heads"] == cfg.num_attention_heads and mixer["n_kv_heads"] == cfg.num_key_value_heads
        assert mixer["head_dim"] == cfg.head_dim and mixer["scale"] == cfg.head_dim ** -0.5
        assert mixer["position"].params["theta"] == cfg.rope_theta
        assert mixer["position"].params["scaling"] == cfg.rope_scaling
        assert spec.layers[-1].part("ffn").params["intermediate_size"] == cfg.intermediate_size
        assert spec.final_norm.params["eps"] == cfg.rms_norm_eps
        assert spec.head.params["tied"] == cfg.tie_word_embeddings
        assert spec.stop_tokens == cfg.eos_token_id
        assert sorted(spec.layers[0].parts) == ["ffn", "mixer", "norm1", "norm2"]
        with pytest.raises(ValueError, match="needs a part in the place 'norm3'"):
            spec.layers[0].part("norm3")
        assert [l.part("mixer").params["window"] for l in spec.layers] == [cfg.window_of_layer(i) for i in range(len(spec.layers))]
