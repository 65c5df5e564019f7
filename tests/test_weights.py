"""Weights: safetensors by name, kept dtypes, one error for everything wrong, random folders."""
import json

import pytest
import torch

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200.config import architecture_of
from longbow_quarrel_b200.engine.model import Model
from longbow_quarrel_b200.parts.base import Runtime
from longbow_quarrel_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_weights,
                                          random_weights, write_random_model, write_safetensors)
from helpers import TINY, make_model_folder
import plain_llama


def _table(name):
    arch = architecture_of(TINY[name])
    cfg = arch.config_from_dict(TINY[name])
    return Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, 64)).weight_table()


def test_table_lists_every_tensor_of_the_architecture():
    table = _table("A")
    assert table["model.embed_tokens.weight"].shape == (256, 64)
    assert table["model.layers.1.self_attn.q_proj.weight"].shape == (64, 64)
    assert table["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert table["model.layers.0.mlp.gate_proj.weight"].shape == (176, 64)
    assert table["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert table["model.layers.0.input_layernorm.weight"].init == "gain"
    assert table["lm_head.weight"].shape == (256, 64) and table["lm_head.weight"].fallback == "model.embed_tokens.weight"
    assert len(table) == 3 + 2 * 9
    assert "lm_head.weight" not in _table("B")     # tied head has no tensor of its own
    assert _table("C")["model.layers.3.self_attn.o_proj.weight"].shape == (80, 240)


def test_round_trip_and_kept_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16), "c": torch.randn(2).to(torch.float16),
               "i": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    write_safetensors(tmp_path / "model.safetensors", tensors)
    plain = plain_llama.read_safetensors(tmp_path / "model.safetensors")     # the plain reader agrees
    for k, v in tensors.items():
        assert torch.equal(plain[k], v)
    from longbow_quarrel_b200.weights import WeightSpec
    table = {"a": WeightSpec((3, 5)), "b": WeightSpec((4, 2)), "c": WeightSpec((2,)), "i": WeightSpec((2, 3), integer=True)}
    out = load_weights(tmp_path, table, "cpu")
    assert out["a"].dtype == torch.float32 and torch.equal(out["a"], tensors["a"])       # 32-bit stays 32-bit
    assert out["b"].dtype == torch.bfloat16 and torch.equal(out["b"], tensors["b"])      # bfloat16 stays
    assert out["c"].dtype == torch.bfloat16                                              # float16 becomes bfloat16
    assert out["i"].dtype == torch.int32 and torch.equal(out["i"].long(), tensors["i"])  # integer tables are int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_folder(tmp_path, "A", seed=1)
    weights = plain_llama.read_safetensors(folder / "model.safetensors")
    del weights["model.layers.0.mlp.up_proj.weight"]
    del weights["model.norm.weight"]
    weights["model.layers.7.extra.weight"] = torch.zeros(2)
    weights["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightsError) as exc:
        load_weights(folder, _table("A"), "cpu")
    err = exc.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 64), (64, 64))]
    text = str(err)
    for piece in ("missing", "unexpected", "wrong shapes", "up_proj", "extra", "expected [32, 64], found [64, 64]"):
        assert piece in text


def test_missing_head_falls_back_to_the_embedding_table(tmp_path):
    folder = make_model_folder(tmp_path, "A", seed=2)
    weights = plain_llama.read_safetensors(folder / "model.safetensors")
    del weights["lm_head.weight"]
    write_safetensors(folder / "model.safetensors", weights)
    out = load_weights(folder, _table("A"), "cpu")
    assert "lm_head.weight" not in out and "model.embed_tokens.weight" in out


def test_a_tied_model_refuses_a_head_tensor(tmp_path):
    folder = make_model_folder(tmp_path, "B", seed=2)
    weights = plain_llama.read_safetensors(folder / "model.safetensors")
    weights["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightsError, match="unexpected.*lm_head.weight"):
        load_weights(folder, _table("B"), "cpu")


def test_unexpected_tensors_may_be_a_warning_instead(tmp_path):
    """Alone they need not stop a load (`unexpected="warn"` names them in a warning, "ignore" says nothing);
    beside another fault they are listed in the one error all the same."""
    folder = make_model_folder(tmp_path, "B", seed=2)
    weights = plain_llama.read_safetensors(folder / "model.safetensors")
    weights["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.bfloat16)
    weights["rotary.inv_freq"] = torch.zeros(16)
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.warns(UserWarning, match="2 tensors.*lm_head.weight, rotary.inv_freq"):
        out = load_weights(folder, _table("B"), "cpu", unexpected="warn")
    assert sorted(out) == sorted(_table("B"))
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        load_weights(folder, _table("B"), "cpu", unexpected="ignore")
    del weights["model.norm.weight"]
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightsError) as exc:
        load_weights(folder, _table("B"), "cpu", unexpected="warn")
    assert exc.value.missing == ["model.norm.weight"] and len(exc.value.unexpected) == 2
    with pytest.raises(ValueError, match="'error', 'warn' or 'ignore'"):
        load_weights(folder, _table("B"), "cpu", unexpected="no")


def test_converting_to_the_models_precision_at_load(tmp_path):
    """Kept as stored by default; `convert_to` rounds matrices to the model's precision and leaves what a
    part computes with in 32-bit (norm gains) as it is stored."""
    folder = make_model_folder(tmp_path, "A", seed=3, dtype=torch.float32)
    table = _table("A")
    stored = load_weights(folder, table, "cpu")
    assert all(t.dtype == torch.float32 for t in stored.values())
    half = load_weights(folder, table, "cpu", convert_to=torch.bfloat16)
    gains = [n for n, spec in table.items() if spec.full_precision]
    assert len(gains) == 2 * 2 + 1
    for name, t in half.items():
        if name in gains:
            assert t.dtype == torch.float32 and torch.equal(t, stored[name])
        else:
            assert t.dtype == torch.bfloat16 and torch.equal(t, stored[name].to(torch.bfloat16))
    # to 32-bit: bfloat16 tensors stay (each of their values is a float32 value), float16 ones are widened
    mixed = {"a": torch.randn(4, 4).to(torch.bfloat16), "b": torch.randn(4, 4).to(torch.float16)}
    write_safetensors(tmp_path / "model.safetensors", mixed)
    from longbow_quarrel_b200.weights import WeightSpec
    out = load_weights(tmp_path, {"a": WeightSpec((4, 4)), "b": WeightSpec((4, 4))}, "cpu", convert_to=torch.float32)
    assert out["a"].dtype == torch.bfloat16 and out["b"].dtype == torch.float32
    assert torch.equal(out["b"], mixed["b"].float())


def test_broken_files_are_refused(tmp_path):
    folder = make_model_folder(tmp_path, "A", seed=3)
    path = folder / "model.safetensors"
    raw = path.read_bytes()
    path.write_bytes(raw[:len(raw) // 2])
    with pytest.raises(SafetensorsError, match="outside the file|truncated"):
        load_weights(folder, _table("A"), "cpu")
    path.write_bytes(b"\x05")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    path.unlink()
    with pytest.raises(SafetensorsError, match="neither"):
        load_weights(folder, _table("A"), "cpu")


def test_sharded_checkpoint(tmp_path):
    folder = make_model_folder(tmp_path, "A", seed=4)
    weights = plain_llama.read_safetensors(folder / "model.safetensors")
    (folder / "model.safetensors").unlink()
    names = sorted(weights)
    parts = {"model-00001-of-00002.safetensors": names[:10], "model-00002-of-00002.safetensors": names[10:]}
    for fname, ns in parts.items():
        write_safetensors(folder / fname, {n: weights[n] for n in ns})
    (folder / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {n: f for f, ns in parts.items() for n in ns}}))
    out = load_weights(folder, _table("A"), "cpu")
    assert all(torch.equal(out[n], weights[n]) for n in names)


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    table = _table("A")
    a = random_weights(table, seed=5, dtype=torch.float32)
    b = random_weights(dict(reversed(list(table.items()))), seed=5, dtype=torch.float32)
    c = random_weights(table, seed=6, dtype=torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    emb = a["model.embed_tokens.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    gain = a["model.norm.weight"]
    assert abs(float(gain.mean()) - 1.0) < 0.1 and 0.03 < float(gain.std()) < 0.2
    folder = write_random_model(tmp_path / "m", TINY["A"], table, seed=5, dtype=torch.bfloat16)
    cfg, stored = plain_llama.load_folder(folder)
    assert cfg["hidden_size"] == 64 and stored["model.norm.weight"].dtype == torch.bfloat16
    assert torch.equal(stored["model.embed_tokens.weight"], emb.to(torch.bfloat16))
