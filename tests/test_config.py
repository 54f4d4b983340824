"""Configuration and registry (CPU)."""
import json

import pytest

from synaptix_b200.config import (ConfigError, Qwen3Config, load_config, register_architecture,
                                  registered_architectures, resolve_architecture)
from tiny import TINY_A, TINY_B, TINY_W


def test_reads_every_size_from_config_json():
    a = Qwen3Config.from_dict(TINY_A)
    b = Qwen3Config.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 6, 2, 32)
    assert (a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps) == (192, 256, 1e4, 1e-6)
    assert (b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps) == (160, 389, 1e6, 1e-5)
    assert a.tie_word_embeddings is True and b.tie_word_embeddings is False
    assert a.eos_token_ids == (7,) and b.eos_token_ids == (11, 12)
    assert a.group_size == 2 and b.group_size == 3
    assert b.q_dim == 192 and b.kv_dim == 64


def test_head_dim_defaults_to_width_over_heads():
    d = dict(TINY_A)
    del d["head_dim"]
    assert Qwen3Config.from_dict(d).head_dim == 16
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="head_dim"):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rms_norm_eps", "rope_theta"])
def test_missing_size_is_an_error(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,match", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"tie_word_embeddings": 1}, "tie_word_embeddings"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
])
def test_validation_errors(patch, match):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict(d)


def test_rope_theta_inside_rope_parameters():
    d = dict(TINY_A)
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(d).rope_theta == 12345.0


def test_windows_per_layer():
    w = Qwen3Config.from_dict(TINY_W)
    assert w.layer_windows == (None, None, 24, 24)
    d = dict(TINY_W)
    d["layer_types"] = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    assert Qwen3Config.from_dict(d).layer_windows == (24, None, None, 24)
    # switched off: every layer sees all keys, whatever sliding_window says
    d = dict(TINY_A, sliding_window=4096, use_sliding_window=False, max_window_layers=1)
    assert Qwen3Config.from_dict(d).layer_windows == (None, None)


def test_round_trip_through_to_dict():
    for src in (TINY_A, TINY_B, TINY_W):
        c = Qwen3Config.from_dict(src)
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_registry_by_architecture_and_model_type(tmp_path):
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_cls is Qwen3Config
    assert resolve_architecture({"model_type": "qwen3"}).config_cls is Qwen3Config
    with pytest.raises(ConfigError, match="registered architectures"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)).vocab_size == 389
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="parse"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="cannot read"):
        load_config(str(tmp_path / "nowhere"))
