"""Weights by name: round trips, dtypes, the one error that lists everything wrong, random-weights mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as P
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.config.registry import architecture, config_from_dict, load_config
from etalii.dllm_b200.weights.loader import WeightError, expected_tensors, load_weights
from etalii.dllm_b200.weights.random_init import random_tensors, write_model, write_random_model
from etalii.dllm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def _spec(config_dict):
    config = config_from_dict(config_dict)
    return config, architecture("llama").build_spec(config)


def _tensors(config_dict, dtype=torch.bfloat16):
    return {k: torch.from_numpy(v).to(dtype) for k, v in P.random_weights(config_dict, 3).items()}


@pytest.mark.parametrize("config_dict", [P.TINY_A, P.TINY_B])
def test_expected_names_are_the_checkpoint_names(config_dict):
    _, spec = _spec(config_dict)
    expected = expected_tensors(spec)
    assert {k: tuple(v.shape) for k, v in expected.items()} == P.tensor_shapes(config_dict)
    assert ("lm_head.weight" in expected) == (not config_dict["tie_word_embeddings"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_round_trip_keeps_storage(tmp_path, dtype):
    tensors = _tensors(P.TINY_B, dtype)
    write_model(str(tmp_path), P.TINY_B, tensors)
    _, spec = _spec(P.TINY_B)
    loaded = load_weights(str(tmp_path), spec)
    want = torch.float32 if dtype == torch.float16 else dtype  # float16 is widened exactly; the others are kept
    for name, tensor in tensors.items():
        assert loaded[name].dtype == want and torch.equal(loaded[name].float(), tensor.float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    tensors = _tensors(P.TINY_A)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    write_model(str(tmp_path), P.TINY_A, tensors)
    _, spec = _spec(P.TINY_A)
    with pytest.raises(WeightError) as info:
        load_weights(str(tmp_path), spec)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.o_proj.bias"]
    assert error.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    text = str(error)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [64, 64]"):
        assert piece in text


def test_tied_head_rules(tmp_path):
    tensors = _tensors(P.TINY_A)
    _, spec = _spec(P.TINY_A)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()  # stored and equal: accepted
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)   # stored rotary table: skipped
    write_model(str(tmp_path), P.TINY_A, tensors)
    assert "lm_head.weight" not in load_weights(str(tmp_path), spec)
    tensors["lm_head.weight"] = tensors["lm_head.weight"] + 1
    write_model(str(tmp_path), P.TINY_A, tensors)
    with pytest.raises(WeightError, match="differs from model.embed_tokens.weight"):
        load_weights(str(tmp_path), spec)
    untied = _tensors(P.TINY_B)
    del untied["lm_head.weight"]
    other = tmp_path / "b"
    write_model(str(other), P.TINY_B, untied)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(str(other), _spec(P.TINY_B)[1])


def test_sharded_checkpoint_and_duplicates(tmp_path):
    tensors = _tensors(P.TINY_A)
    names = list(tensors)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {n: tensors[n] for n in first})
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {n: tensors[n] for n in second})
    index = {"weight_map": {**{n: "model-00001-of-00002.safetensors" for n in first},
                            **{n: "model-00002-of-00002.safetensors" for n in second}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text(json.dumps(P.TINY_A))
    _, spec = _spec(P.TINY_A)
    loaded = load_weights(str(tmp_path), spec)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {n: tensors[n] for n in second + first[:1]})
    with pytest.raises(WeightError, match="more than one file"):
        load_weights(str(tmp_path), spec)


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError, match="no safetensors"):
        load_weights(str(tmp_path), _spec(P.TINY_A)[1])
    path = tmp_path / "model.safetensors"
    path.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{}")
    with pytest.raises(SafetensorsError, match="header runs past"):
        SafetensorsFile(str(path))
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad offsets"):
        SafetensorsFile(str(path))
    header = json.dumps({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                         "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    path.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="overlap"):
        SafetensorsFile(str(path))


def test_random_weights_mode(tmp_path):
    config = config_from_dict(P.TINY_B)
    folder = write_random_model(str(tmp_path / "m"), config, seed=4)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert load_config(folder) == config
    spec = architecture("llama").build_spec(config)
    loaded = load_weights(folder, spec)
    again = random_tensors(config, 4)
    other = random_tensors(config, 5)
    for name, tensor in loaded.items():
        assert tensor.dtype == torch.bfloat16 and torch.equal(tensor, again[name])
        assert not torch.equal(tensor, other[name])
    matrix = loaded["model.layers.1.mlp.down_proj.weight"].float()
    norm = loaded["model.layers.2.input_layernorm.weight"].float()
    assert abs(matrix.std().item() - 0.02) < 0.002 and abs(matrix.mean().item()) < 0.002
    assert abs(norm.mean().item() - 1.0) < 0.01 and norm.std().item() < 0.03
    # a tensor's numbers depend on (seed, name) only: the tied model's embedding equals the untied one's
    tied = random_tensors(config_from_dict(dict(P.TINY_B, tie_word_embeddings=True)), 4)
    assert "lm_head.weight" not in tied and torch.equal(tied["model.embed_tokens.weight"], again["model.embed_tokens.weight"])
