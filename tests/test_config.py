"""Configuration and registry (no GPU)."""

import json

import pytest

from helpers import TINY_CONFIGS
from quantinfer_b200.config import (Qwen3Config, architectures, config_from_dict, load_config,
                                    register_architecture)
from quantinfer_b200.errors import ConfigError


def test_parse_and_derived_sizes():
    cfg = config_from_dict(TINY_CONFIGS["B"])
    assert isinstance(cfg, Qwen3Config)
    assert cfg.effective_head_dim == 32 and cfg.query_projection_size == 256
    assert cfg.key_value_projection_size == 32 and cfg.kv_group_size == 8
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and not cfg.tie_word_embeddings


def test_defaults_of_absent_keys():
    d = dict(TINY_CONFIGS["A"])
    for k in ("head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        d.pop(k)
    cfg = config_from_dict(d)
    assert cfg.effective_head_dim == 64 // 4
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1_000_000.0 and cfg.tie_word_embeddings is False


def test_unknown_keys_are_ignored():
    d = dict(TINY_CONFIGS["A"], some_future_key=3, attention_dropout=0.0)
    assert config_from_dict(d).vocab_size == 256


@pytest.mark.parametrize("change, message", [
    ({"vocab_size": 0}, "greater than zero"),
    ({"num_attention_heads": 5}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": float("nan")}, "finite"),
    ({"rms_norm_eps": 0.0}, "positive"),
    ({"rope_theta": -1.0}, "positive"),
    ({"sliding_window": 128}, "sliding"),
    ({"use_sliding_window": True}, "sliding"),
    ({"rope_scaling": {"type": "yarn"}}, "scaling"),
    ({"hidden_size": "64"}, "integer"),
    ({"num_hidden_layers": 2.5}, "integer"),
    ({"tie_word_embeddings": 1}, "true or false"),
    ({"model_type": "llama"}, "model_type"),
])
def test_validation_errors(change, message):
    d = dict(TINY_CONFIGS["A"], **change)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_missing_key_is_named():
    d = dict(TINY_CONFIGS["A"])
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(d)


def test_head_dim_absent_needs_divisible_hidden():
    d = dict(TINY_CONFIGS["A"], hidden_size=66)
    del d["head_dim"]
    with pytest.raises(ConfigError, match="divisible by attention heads"):
        config_from_dict(d)


def test_registry_selects_by_architecture(tmp_path):
    assert "Qwen3ForCausalLM" in architectures()
    with pytest.raises(ConfigError, match="unsupported architecture 'LlamaForCausalLM'"):
        config_from_dict(dict(TINY_CONFIGS["A"], architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_CONFIGS["A"].items() if k != "architectures"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_CONFIGS["C"]))
    assert load_config(tmp_path).hidden_size == 168
    with pytest.raises(ConfigError, match="does not exist"):
        load_config(tmp_path / "nowhere")


def test_registering_another_architecture():
    class ToyConfig:
        @classmethod
        def from_dict(cls, d):
            return cls()

    register_architecture("ToyForCausalLM", ToyConfig)
    assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), ToyConfig)


def test_model_spec_is_data():
    cfg = config_from_dict(TINY_CONFIGS["B"])
    spec = cfg.to_model_spec()
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    a = spec.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.qk_norm, a.window) == (8, 1, 32, True, None)
    assert a.position.theta == 1e6 and a.position.rotary_dim == 32 and a.position.max_positions == 256
    assert spec.layers[0].ffn.intermediate_size == 224 and spec.final_norm.eps == 1e-5
    assert spec.head.tied is False and spec.cache_entries() == 3


def test_round_trip_through_to_dict():
    cfg = config_from_dict(TINY_CONFIGS["C"])
    assert config_from_dict(cfg.to_dict()) == cfg
