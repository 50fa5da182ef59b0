"""Configuration and registry: keys come from config.json, nothing is defaulted, names map to models."""

import json

import pytest

from gtar_kimik3_public_b200.config import ConfigError, TransformerConfig
from gtar_kimik3_public_b200.registry import architecture, config_from_dict, config_from_file, known_architectures
from tests.tiny_configs import TINY_A, TINY_B


def test_both_names_reach_the_same_architecture():
    assert "transformer" in known_architectures() and "Qwen3ForCausalLM" in known_architectures()
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, TransformerConfig) and isinstance(b, TransformerConfig)
    assert architecture("transformer").build_plan is architecture("Qwen3ForCausalLM").build_plan
    assert (a.head_dim, a.num_key_value_heads, a.tie_word_embeddings) == (16, 2, True)
    assert (b.rope_theta, b.rms_norm_eps, b.tie_word_embeddings) == (1e6, 1e-5, False)


def test_missing_and_unknown_keys_are_listed_together():
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rope_theta")}
    raw["num_experts"] = 4
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    text = str(err.value)
    assert "head_dim" in text and "rope_theta" in text and "num_experts" in text


def test_no_size_is_defaulted():
    required = set(TransformerConfig.required_keys())
    assert {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"} <= required


@pytest.mark.parametrize("key,value", [
    ("num_key_value_heads", 3), ("head_dim", 15), ("head_dim", 12), ("hidden_size", 0), ("rms_norm_eps", 0.0), ("eos_token_id", 9999),
    ("vocab_size", 2.5), ("tie_word_embeddings", 1),
])
def test_bad_values_are_refused(key, value):
    with pytest.raises(ConfigError):
        config_from_dict({**TINY_A, key: value})


def test_keys_the_architecture_does_not_vary():
    config_from_dict({**TINY_A, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"})
    with pytest.raises(ConfigError):
        config_from_dict({**TINY_A, "hidden_act": "gelu"})
    with pytest.raises(ConfigError):
        config_from_dict({**TINY_A, "attention_bias": True})


def test_unknown_architecture_names_the_known_ones():
    with pytest.raises(ConfigError) as err:
        config_from_dict({**TINY_A, "arch": "mamba"})
    assert "transformer" in str(err.value)
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "arch"})


def test_reference_nested_file_and_round_trip(tmp_path):
    nested = {"arch": "transformer", "model": {k: v for k, v in TINY_A.items() if k not in ("arch", "vocab_size")},
              "train": {"seq_len": 128}}
    path = tmp_path / "nested.json"
    path.write_text(json.dumps(nested))
    with pytest.raises(ConfigError):  # the reference's files carry no vocab_size
        config_from_file(path)
    config = config_from_file(path, {"vocab_size": 256})
    assert config == config_from_dict(TINY_A)
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    assert config_from_file(tmp_path) == config
