import json

import pytest

from rosellm_b200.config import (ConfigError, EngineConfig, GPT2Config, ModelConfig, load_config, parse_config,
                                 register_architecture, registered_architectures, unregister_architecture)

RAW = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 3, "n_embd": 96, "n_head": 3,
       "n_inner": 320, "vocab_size": 1000, "n_positions": 256, "layer_norm_epsilon": 1e-6,
       "activation_function": "gelu"}


def test_gpt2_keys_are_read():
    c = parse_config(RAW)
    assert isinstance(c, GPT2Config)
    assert (c.n_layer, c.n_embd, c.n_head, c.n_inner, c.vocab_size, c.n_positions) == (3, 96, 3, 320, 1000, 256)
    assert c.layer_norm_epsilon == 1e-6 and c.activation_function == "gelu" and c.head_dim == 32
    assert parse_config(c.to_dict()) == c


def test_inner_size_defaults_to_four_times_width_and_positions_fallback():
    raw = dict(RAW, n_inner=None)
    del raw["n_positions"]
    raw["max_position_embeddings"] = 77
    c = parse_config(raw)
    assert c.n_inner == 4 * 96 and c.n_positions == 77


@pytest.mark.parametrize("key", ["n_layer", "n_embd", "n_head", "vocab_size", "n_positions"])
def test_sizes_are_required(key):
    raw = dict(RAW)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        parse_config(raw)


@pytest.mark.parametrize("patch,match", [
    ({"n_head": 5}, "not divisible"), ({"activation_function": "relu"}, "activation_function"),
    ({"scale_attn_by_inverse_layer_idx": True}, "scale_attn_by_inverse_layer_idx"),
    ({"scale_attn_weights": False}, "scale_attn_weights"), ({"tie_word_embeddings": False}, "tie_word_embeddings"),
    ({"n_layer": "3"}, "must be int"), ({"n_embd": 0}, "positive"),
])
def test_unsupported_values_are_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        parse_config(dict(RAW, **patch))


def test_registry_by_architecture_name_and_model_type(tmp_path):
    assert "GPT2LMHeadModel" in registered_architectures()
    with pytest.raises(ConfigError, match="unknown architecture"):
        parse_config(dict(RAW, architectures=["LlamaForCausalLM"]))
    raw = dict(RAW)
    del raw["architectures"]
    assert isinstance(parse_config(raw), GPT2Config)  # model_type stands in
    (tmp_path / "config.json").write_text(json.dumps(RAW))
    assert load_config(str(tmp_path)).n_embd == 96
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))


def test_another_architecture_is_one_registration():
    class ToyConfig(ModelConfig):
        architecture = "ToyLM"

        @classmethod
        def from_dict(cls, raw):
            return cls()

    register_architecture("ToyLM", ToyConfig, lambda c: None)
    try:
        assert isinstance(parse_config({"architectures": ["ToyLM"]}), ToyConfig)
        with pytest.raises(ConfigError, match="already registered"):
            register_architecture("ToyLM", ToyConfig, lambda c: None)
    finally:
        unregister_architecture("ToyLM")


def test_engine_config():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ConfigError):
        EngineConfig(dtype="float16")
    with pytest.raises(ConfigError):
        EngineConfig(page_size=0)
