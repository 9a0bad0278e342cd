"""Configuration, registry, safetensors container, weight errors and the random-weights mode (no GPU)."""
from __future__ import annotations

import json
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C
from stride_b200.config import ConfigError, LlamaConfig, registered_architectures, resolve_architecture
from stride_b200.weights.loader import WeightsError, check_plan, load_weights, storage_dtype
from stride_b200.weights.random_init import model_plan, random_tensors, write_random_model
from stride_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def test_config_defaults_and_keys():
    c = LlamaConfig.from_dict({"hidden_size": 96, "intermediate_size": 100, "num_hidden_layers": 2,
                               "num_attention_heads": 6, "vocab_size": 50})
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (6, 16, 1e-5, 10000.0)
    assert c.rope_scaling.rope_type == "default" and c.eos_token_ids == () and c.tie_word_embeddings is None
    b = LlamaConfig.from_dict(TINY_B)
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.original_max_position_embeddings == 64
    assert b.num_attention_heads // b.num_key_value_heads == 3 and b.tie_word_embeddings is False
    cc = LlamaConfig.from_dict(TINY_C)           # "type" instead of "rope_type", head_dim != hidden / heads
    assert cc.rope_scaling.rope_type == "llama3" and cc.rope_scaling.factor == 8.0 and cc.head_dim == 48
    assert LlamaConfig.from_dict({**TINY_A, "eos_token_id": 7}).eos_token_ids == (7,)
    assert LlamaConfig.from_dict({**TINY_A, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)
    assert LlamaConfig.from_dict(b.to_dict()) == LlamaConfig.from_dict({**b.to_dict()})
    assert LlamaConfig.from_dict(b.to_dict()).rope_scaling == b.rope_scaling


@pytest.mark.parametrize("patch,needle", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": 0}, "vocab_size"), ({"num_hidden_layers": "2"}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"head_dim": 15}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn"}}, "yarn"), ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"), ({"hidden_act": "gelu"}, "gelu"), ({"rms_norm_eps": 0.0}, "rms_norm_eps")])
def test_config_errors_name_the_key(patch, needle):
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict({**TINY_A, **patch})
    assert needle in str(e.value)


def test_registry():
    assert "LlamaForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["MambaForCausalLM"]})
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        resolve_architecture({})


def test_model_spec_is_data():
    arch = resolve_architecture(TINY_B)
    spec = arch.model_spec(arch.parse_config(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "attention" and m.params["num_kv_heads"] == 2 and m.params["position"].params["theta"] == 500000.0
    assert m.tensors["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert spec.layers[2].feed_forward.params == {"hidden_size": 192, "intermediate_size": 320}
    assert spec.final_norm.params["eps"] == 1e-6 and spec.head.params["tied"] is False


def test_safetensors_round_trip_and_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t, {"k": "v"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == list("abcde") and f.shape("a") == (3, 5) and f.dtype("c") == torch.int64
    for k in t:
        assert torch.equal(f.get(k), t[k])
    assert storage_dtype(torch.bfloat16, False) == torch.bfloat16 and storage_dtype(torch.float16, False) == torch.float32
    assert storage_dtype(torch.float32, False) == torch.float32 and storage_dtype(torch.int64, False) == torch.int32
    with pytest.raises(SafetensorsError, match="missing tensor 'zz'"):
        f.get("zz")


def test_safetensors_rejects_broken_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(tmp_path / "none.safetensors")
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="overruns"):
        SafetensorsFile(p)
    h = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad offsets for tensor 'w'"):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    model = write_random_model(tmp_path / "m", TINY_B, 2)
    plan = model_plan(TINY_B)
    tensors = {n: SafetensorsFile(model / "model.safetensors").get(n).clone() for n in plan}
    assert set(load_weights(model, plan, "cpu")) == set(plan)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(32, 192, dtype=torch.bfloat16)
    write_safetensors(model / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as e:
        load_weights(model, plan, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == [("model.layers.2.self_attn.k_proj.weight", (32, 192), (64, 192))]
    for needle in ("up_proj", "model.norm.weight", "q_proj.bias", "[32, 192]", "[64, 192]"):
        assert needle in str(err)
    check_plan(plan, {n: plan[n].shape for n in plan}, "x")      # a full match passes


def test_tied_and_untied_heads():
    assert "lm_head.weight" in model_plan(TINY_B) and not model_plan(TINY_B)["lm_head.weight"].optional
    assert "lm_head.weight" not in model_plan(TINY_A)
    c_plan = model_plan(TINY_C)                                 # no tie key: the file decides
    assert c_plan["lm_head.weight"].optional
    assert "lm_head.weight" not in random_tensors(TINY_C, 1) and "lm_head.weight" in random_tensors(TINY_B, 1)


def test_random_weights_are_seeded_per_tensor(tmp_path):
    a, b = random_tensors(TINY_A, 0), random_tensors(TINY_A, 0)
    c = random_tensors(TINY_A, 1)
    for n in a:
        assert torch.equal(a[n], b[n]) and a[n].dtype == torch.bfloat16
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    # a tensor's values depend on (seed, name) only, not on the other tensors of the model
    fewer = random_tensors({**TINY_A, "num_hidden_layers": 1}, 0)
    assert torch.equal(fewer["model.layers.0.mlp.down_proj.weight"], a["model.layers.0.mlp.down_proj.weight"])
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.003 and abs(float(a["model.norm.weight"].float().mean()) - 1.0) < 0.1
    d = write_random_model(tmp_path / "m", TINY_A, 0)
    assert json.loads((d / "config.json").read_text())["hidden_size"] == 64
    f = SafetensorsFile(d / "model.safetensors")
    assert torch.equal(f.get("model.embed_tokens.weight"), a["model.embed_tokens.weight"])
    f32 = random_tensors(TINY_A, 0, dtype=torch.float32)
    assert f32["model.norm.weight"].dtype == torch.float32


def test_sharded_checkpoints_load_like_the_single_file(tmp_path):
    """A model folder with `model.safetensors.index.json` and two shards gives the same tensors as the single file;
    an index that names a missing shard, or a tensor its shard does not hold, is an error that says so."""
    import json

    from stride_b200.weights.safetensors_io import SafetensorsError
    model = write_random_model(tmp_path / "m", TINY_B, 2)
    plan = model_plan(TINY_B)
    whole = load_weights(model, plan, "cpu")
    names = sorted(whole)
    halves = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    sharded = tmp_path / "s"
    sharded.mkdir()
    (sharded / "config.json").write_text((model / "config.json").read_text())
    for shard, keys in halves.items():
        write_safetensors(sharded / shard, {n: whole[n] for n in keys})
    index = {"metadata": {}, "weight_map": {n: shard for shard, keys in halves.items() for n in keys}}
    (sharded / "model.safetensors.index.json").write_text(json.dumps(index))
    again = load_weights(sharded, plan, "cpu")
    assert set(again) == set(whole) and all(torch.equal(again[n], whole[n]) and again[n].dtype == whole[n].dtype for n in whole)
    # one error for all that is wrong, as with a single file
    del index["weight_map"]["model.norm.weight"]
    (sharded / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightsError) as e:
        load_weights(sharded, plan, "cpu")
    assert e.value.missing == ["model.norm.weight"]
    index["weight_map"]["model.norm.weight"] = "model-00001-of-00002.safetensors"       # it lives in the other shard
    (sharded / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightsError, match="which it does not"):
        load_weights(sharded, plan, "cpu")
    index["weight_map"]["model.norm.weight"] = "model-00003-of-00002.safetensors"
    (sharded / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError, match="cannot open"):
        load_weights(sharded, plan, "cpu")
    (sharded / "model.safetensors.index.json").write_text("[1, 2]")
    with pytest.raises(WeightsError, match="not a shard index"):
        load_weights(sharded, plan, "cpu")


def test_float16_checkpoints_are_widened_exactly(tmp_path):
    """A float16 tensor is kept as float32 (exact), never as bfloat16, which would drop mantissa bits silently."""
    plan = model_plan(TINY_A)
    tensors = random_tensors(TINY_A, 3, dtype=torch.float32)
    half = {n: t.to(torch.float16) for n, t in tensors.items()}
    (tmp_path / "config.json").write_text("{}")
    write_safetensors(tmp_path / "model.safetensors", half)
    got = load_weights(tmp_path, plan, "cpu")
    for n, t in half.items():
        assert got[n].dtype == torch.float32 and torch.equal(got[n], t.to(torch.float32))
