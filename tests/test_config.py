"""Configuration and registry (no GPU)."""
import json

import pytest

import plain_llama as P
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.config.llama import LlamaConfig, RopeScaling
from etalii.dllm_b200.config.registry import (ConfigError, config_from_dict, load_config, register_architecture,
                                              supported_architectures, unregister_architecture)


def test_tiny_configs_parse_and_differ_in_everything():
    a, b = config_from_dict(P.TINY_A), config_from_dict(P.TINY_B)
    assert isinstance(a, LlamaConfig) and isinstance(b, LlamaConfig)
    for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                 "num_key_value_heads", "head_dim", "max_position_embeddings", "rms_norm_eps", "rope_theta",
                 "rope_scaling", "tie_word_embeddings", "eos_token_ids"):
        assert getattr(a, name) != getattr(b, name), name
    assert b.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    assert a.eos_token_ids == (2,) and b.eos_token_ids == (3, 5)


def test_defaults_follow_the_reference():
    config = config_from_dict({"model_type": "llama", "vocab_size": 10, "hidden_size": 48, "intermediate_size": 20,
                               "num_hidden_layers": 1, "num_attention_heads": 3})
    assert config.num_key_value_heads == 3 and config.head_dim == 16
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 10000.0 and config.max_position_embeddings == 2048
    assert config.tie_word_embeddings is False and config.rope_scaling is None and config.eos_token_ids == ()


def test_round_trip_through_config_json(tmp_path):
    for source in (P.TINY_A, P.TINY_B):
        config = config_from_dict(source)
        (tmp_path / "config.json").write_text(json.dumps(config.to_hf()))
        assert load_config(str(tmp_path)) == config


def test_generation_config_adds_stop_ids(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(P.TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 9]}))
    assert load_config(str(tmp_path)).eos_token_ids == (2, 9)


def test_rope_parameters_layout_and_legacy_type_key():
    base = {k: v for k, v in P.TINY_B.items() if k not in ("rope_scaling", "rope_theta")}
    new = dict(base, rope_parameters={"rope_theta": 500000.0, **P.TINY_B["rope_scaling"]})
    assert config_from_dict(new) == config_from_dict(P.TINY_B)
    legacy = dict(P.TINY_B, rope_scaling={"type": "linear", "factor": 2.0})
    assert config_from_dict(legacy).rope_scaling == RopeScaling("linear", 2.0)
    assert config_from_dict(dict(P.TINY_B, rope_scaling={"rope_type": "default"})).rope_scaling is None


@pytest.mark.parametrize("change,message", [
    ({"model_type": "gpt2"}, "not supported (supported: "),
    ({"hidden_act": "gelu"}, "activation"),
    ({"mlp_bias": True}, "MLP biases"),
    ({"attention_bias": True}, "attention biases"),
    ({"clip_qkv": 8.0}, "clip_qkv"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "RoPE scaling 'yarn'"),
    ({"num_key_value_heads": 3}, "multiple of num_key_value_heads"),
    ({"head_dim": 15}, "head_dim must be even"),
    ({"vocab_size": 0}, "vocab_size must be positive"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_refusals(change, message):
    with pytest.raises(ConfigError, match=message.replace("(", r"\(")):
        config_from_dict(dict(P.TINY_A, **change))


def test_missing_key_and_missing_file(tmp_path):
    broken = {k: v for k, v in P.TINY_A.items() if k != "intermediate_size"}
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(broken)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))


def test_registry_is_open():
    class ToyConfig:
        model_type = "toy"

        @classmethod
        def from_hf(cls, config, generation=None):
            return cls()

    assert "llama" in supported_architectures()
    register_architecture("toy", ToyConfig, lambda config: None)
    try:
        assert isinstance(config_from_dict({"model_type": "toy"}), ToyConfig)
        with pytest.raises(ValueError):
            register_architecture("toy", ToyConfig, lambda config: None)
    finally:
        unregister_architecture("toy")
    with pytest.raises(ConfigError):
        config_from_dict({"model_type": "toy"})
