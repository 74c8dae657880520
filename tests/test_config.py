"""Configuration and registry. No GPU."""

import json

import pytest

import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from semantic_aware_adaptive_kv_cache_precision_b200.config import (ConfigError, LayerCall,
                                                                     Qwen2Config)
from conftest import TINY_A, TINY_B, TINY_W


def test_every_size_comes_from_config_json():
    a, b = Qwen2Config.from_dict(TINY_A), Qwen2Config.from_dict(TINY_B)
    assert (a.head_dim, b.head_dim) == (16, 32)
    sa, sb = a.model_spec(), b.model_spec()
    assert len(sa.blocks) == 2 and len(sb.blocks) == 3
    assert sa.blocks[0].mixer.kv_heads == 2 and sb.blocks[0].mixer.kv_heads == 1
    assert sa.blocks[0].mixer_norm.eps == 1e-6 and sb.blocks[0].mixer_norm.eps == 1e-5
    assert sa.blocks[0].mixer.position.theta == 1e4 and sb.blocks[0].mixer.position.theta == 1e6
    assert sa.tie_head and not sb.tie_head
    assert sa.blocks[1].ffn.intermediate == 176 and sb.blocks[1].ffn.intermediate == 352
    assert sa.stop_token_ids == (7,) and sb.stop_token_ids == (11, 13)
    assert sa.run_order == (LayerCall(0, 0), LayerCall(1, 1))
    assert abs(sb.blocks[0].mixer.scale - 32 ** -0.5) < 1e-12


def test_window_keys_choose_windowed_layers():
    spec = Qwen2Config.from_dict(TINY_W).model_spec()
    assert [b.mixer.window for b in spec.blocks] == [None, 70, 70, 70]
    assert spec.blocks[0].mixer.head_dim == 48
    off = dict(TINY_W, use_sliding_window=False)
    assert all(b.mixer.window is None for b in Qwen2Config.from_dict(off).model_spec().blocks)


def test_all_problems_are_named_at_once():
    bad = dict(TINY_A, num_key_value_heads=3, hidden_act="gelu", rope_scaling={"type": "yarn"})
    del bad["vocab_size"]
    with pytest.raises(ConfigError) as err:
        Qwen2Config.from_dict(bad)
    assert "vocab_size" in str(err.value)
    bad["vocab_size"] = 10
    with pytest.raises(ConfigError) as err:
        Qwen2Config.from_dict(bad)
    text = str(err.value)
    assert "num_key_value_heads" in text and "gelu" in text and "rope_scaling" in text


def test_wrong_types_are_refused():
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen2Config.from_dict(dict(TINY_A, hidden_size="64"))
    with pytest.raises(ConfigError, match="odd"):
        Qwen2Config.from_dict(dict(TINY_A, head_dim=15))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(dict(TINY_A, use_sliding_window=True, sliding_window=None))


def test_registry_by_architecture_name(tmp_path):
    assert "Qwen2ForCausalLM" in sakv.known_architectures()
    assert isinstance(sakv.config_from_dict(TINY_A), Qwen2Config)
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*Qwen2ForCausalLM"):
        sakv.config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        sakv.config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="config.json"):
        sakv.config_from_folder(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        sakv.config_from_folder(tmp_path)


def test_config_round_trip(tmp_path):
    for raw in (TINY_A, TINY_B, TINY_W):
        config = Qwen2Config.from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
        assert sakv.config_from_folder(tmp_path) == config


def test_a_new_architecture_registers_without_touching_the_package():
    class Toy:
        @classmethod
        def from_dict(cls, raw):
            return cls()

    sakv.register_architecture("ToyForTests", Toy)
    try:
        assert isinstance(sakv.config_from_dict({"architectures": ["ToyForTests"]}), Toy)
    finally:
        from semantic_aware_adaptive_kv_cache_precision_b200.config import registry
        registry._ARCHITECTURES.pop("ToyForTests")
