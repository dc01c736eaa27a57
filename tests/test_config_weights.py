"""Configuration, registry, safetensors and weight errors (no GPU)."""

import json
import struct

import pytest
import torch

from tiny import TINY_A, TINY_B, TINY_C, make_folder

from models_b200.config import ConfigError, LlamaConfig, config_from_dict, known_architectures, load_config
from models_b200.engine.model import parameter_requests
from models_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, random_tensors,
                                 write_safetensors)


def test_llama_config_reads_its_own_keys():
    c = config_from_dict(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (32, 256, 320, 256)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (5, 7)
    assert (c.query_dim, c.key_dim, c.value_dim, c.attention_output_dim) == (96, 32, 32, 96)
    assert config_from_dict(c.to_dict()) == c  # what random-weights mode writes reads back the same


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps",
                                                        "max_position_embeddings")}
    c = config_from_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads  # absent: as many kv heads as heads
    assert c.head_dim == 16  # hidden / heads
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5 and c.max_position_embeddings == 2048


def test_rope_parameters_form_is_read_too():
    raw = dict(TINY_B)
    scaling = raw.pop("rope_scaling")
    theta = raw.pop("rope_theta")
    raw["rope_parameters"] = dict(scaling, rope_theta=theta)
    assert config_from_dict(raw) == config_from_dict(TINY_B)


@pytest.mark.parametrize("change,message", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_attention_heads": 4, "num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"rms_norm_eps": float("nan")}, "rms_norm_eps"),
    ({"eos_token_id": 100000}, "vocabulary"),
    ({"vocab_size": "many"}, "vocab_size"),
])
def test_bad_configs_are_refused_by_name(change, message):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_registry_lists_what_is_built():
    assert known_architectures() == ["LlamaForCausalLM"]
    with pytest.raises(ConfigError, match="MistralForCausalLM.*LlamaForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["MistralForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_model_spec_has_a_part_per_layer_and_names_every_tensor():
    spec = config_from_dict(TINY_C).model_spec()
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    assert spec.layers[0].mixer.head_dim == 48 and spec.layers[0].mixer.bias
    names = parameter_requests(spec)
    assert "model.layers.1.self_attn.k_proj.bias" in names and "lm_head.weight" in names
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (80, 136)
    tied = parameter_requests(config_from_dict(TINY_A).model_spec())
    assert "lm_head.weight" not in tied


def test_random_model_folder_round_trip(tmp_path):
    folder = make_folder(TINY_B, 5, tmp_path)
    assert sorted(p.name for p in folder.iterdir()) == ["config.json", "model.safetensors"]
    config = load_config(folder)
    requests = parameter_requests(config.model_spec())
    tensors = load_tensors(folder, requests)
    assert set(tensors) == set(requests)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    again = random_tensors(requests, 5)
    assert all(torch.equal(tensors[n], again[n]) for n in requests)  # seed and name decide the values
    other = random_tensors(requests, 6)
    assert not torch.equal(tensors["model.norm.weight"], other["model.norm.weight"])
    gains = tensors["model.norm.weight"].float()
    assert abs(float(gains.mean()) - 1.0) < 0.1
    assert float(tensors["model.embed_tokens.weight"].float().std()) == pytest.approx(0.02, rel=0.1)


def test_32_bit_tensors_stay_32_bit_and_integers_become_int32(tmp_path):
    path = tmp_path / "t.safetensors"
    write_safetensors(path, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.ones(4, dtype=torch.bfloat16),
                             "c": torch.arange(5, dtype=torch.int64), "d": torch.ones(2, dtype=torch.float16)})
    with SafetensorsFile(path) as f:
        assert f.tensor("a").dtype == torch.float32 and f.tensor("a")[1, 2] == 5
        assert f.tensor("b").dtype == torch.bfloat16
        assert f.tensor("c").dtype == torch.int32 and f.tensor("c").tolist() == [0, 1, 2, 3, 4]
        assert f.tensor("d").dtype == torch.bfloat16
        with pytest.raises(SafetensorsError, match="not found: zz"):
            f.tensor("zz")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = config_from_dict(TINY_A)
    requests = parameter_requests(config.model_spec())
    tensors = random_tensors(requests, 1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)  # tied model: not expected
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    folder = tmp_path / "broken"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as info:
        load_tensors(folder, requests)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["lm_head.weight"]
    assert [w[0] for w in error.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    text = str(error)
    for needle in ("missing (2)", "model.norm.weight", "unexpected (1)", "lm_head.weight", "wrong shape (1)",
                   "is [64, 32], the model needs [64, 64]"):
        assert needle in text


def test_truncated_and_malformed_files(tmp_path):
    good = tmp_path / "good.safetensors"
    write_safetensors(good, {"a": torch.zeros(8, 8)})
    raw = good.read_bytes()
    cut = tmp_path / "cut.safetensors"
    cut.write_bytes(raw[:-10])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(cut)
    tiny = tmp_path / "tiny.safetensors"
    tiny.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(tiny)
    header = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 12 bytes"):
        SafetensorsFile(bad)
    dup = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    twice = tmp_path / "twice.safetensors"
    twice.write_bytes(struct.pack("<Q", len(dup)) + dup + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="twice"):
        SafetensorsFile(twice)
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        load_tensors(tmp_path, {})
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_config(tmp_path)


def test_sharded_folder_with_index(tmp_path):
    config = config_from_dict(TINY_A)
    requests = parameter_requests(config.model_spec())
    tensors = random_tensors(requests, 2)
    names = sorted(tensors)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: tensors[n] for n in first})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in second})
    weight_map = {n: "model-00001-of-00002.safetensors" for n in first}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in second})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    loaded = load_tensors(tmp_path, requests)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)


def test_random_values_are_normal_and_keyed_by_seed_and_name():
    """The generator behind random-weights mode: standard normal moments, a value for every index
    whatever the count (element i does not depend on how many are drawn), other values under another key."""
    import numpy as np

    from models_b200.weights.philox_normal import normal_float32, tensor_key

    key = tensor_key(3, "model.embed_tokens.weight")
    assert key == tensor_key(3, "model.embed_tokens.weight") and key != tensor_key(4, "model.embed_tokens.weight")
    assert key != tensor_key(3, "model.norm.weight")
    z = normal_float32(1_000_003, key, 0.0, 1.0).astype(np.float64)
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1.0) < 5e-3
    assert abs(((z - z.mean()) ** 3).mean()) < 2e-2  # skewness 0
    assert abs(((z - z.mean()) ** 4).mean() / z.var() ** 2 - 3.0) < 5e-2  # kurtosis 3: tails as a normal's
    assert np.isfinite(z).all() and z.max() > 4.0 and z.min() < -4.0
    assert abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 5e-3  # the two values of a pair, and neighbours, are uncorrelated
    short = normal_float32(1001, key, 0.0, 1.0)
    assert np.array_equal(short, z[:1001].astype(np.float32))
    shifted = normal_float32(1001, key, 1.0, 0.1)
    assert np.array_equal(shifted, (short * np.float32(0.1) + np.float32(1.0)).astype(np.float32))
    assert not np.array_equal(short, normal_float32(1001, tensor_key(3, "model.norm.weight"), 0.0, 1.0))


def test_recomputed_buffers_and_a_tied_models_stored_output_matrix(tmp_path):
    """What a checkpoint may hold beyond the model's tensors: rotation-frequency buffers (ignored: they
    are recomputed), and for a tied model the output matrix itself -- accepted when it repeats the
    embedding table, refused when the two differ.  Any other unknown tensor is still an error."""
    config = config_from_dict(TINY_A)
    spec = config.model_spec()
    requests = parameter_requests(spec)
    tensors = random_tensors(requests, 1)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    folder = tmp_path / "with_extras"
    folder.mkdir()
    write_safetensors(folder / "model.safetensors", tensors)
    loaded = load_tensors(folder, requests, spec.ignored_tensors, spec.duplicate_tensors)
    assert set(loaded) == set(requests)
    with pytest.raises(WeightsError, match="unexpected"):  # without the architecture's word for it, both are unknown
        load_tensors(folder, requests)
    tensors["lm_head.weight"][3, 5] += 1.0
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError, match="the two differ"):
        load_tensors(folder, requests, spec.ignored_tensors, spec.duplicate_tensors)
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.something_else"] = torch.ones(8)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError, match="something_else"):
        load_tensors(folder, requests, spec.ignored_tensors, spec.duplicate_tensors)
    untied = config_from_dict(TINY_B).model_spec()
    assert untied.duplicate_tensors == {}  # an untied model needs its output matrix; nothing stands in for it
