"""Configuration and registry (no device)."""
import copy
import json

import pytest

from conftest import TINY
from sonicboom_b200.config import (ConfigError, Qwen2Config, ScheduleEntry, lookup,
                                   read_config_json, register_architecture, spec_from_config_dict)


def test_every_size_comes_from_the_file():
    for name, d in TINY.items():
        cfg, spec = spec_from_config_dict(d)
        assert isinstance(cfg, Qwen2Config)
        assert spec.width == d["hidden_size"] and spec.vocab == d["vocab_size"]
        assert len(spec.layers) == d["num_hidden_layers"] == len(spec.schedule)
        hd = d.get("head_dim", d["hidden_size"] // d["num_attention_heads"])
        for l in spec.layers:
            assert l.mixer.n_heads == d["num_attention_heads"]
            assert l.mixer.n_kv_heads == d["num_key_value_heads"]
            assert l.mixer.head_dim == hd == l.mixer.position.head_dim
            assert l.mixer.position.theta == d["rope_theta"]
            assert l.mixer_norm.eps == d["rms_norm_eps"] == l.feed_forward_norm.eps
            assert l.feed_forward.intermediate == d["intermediate_size"]
            assert l.mixer.qkv_bias and not l.mixer.out_bias
            assert abs(l.mixer.scale - hd ** -0.5) < 1e-7
        assert (spec.head_tensor is None) == d["tie_word_embeddings"]
        assert spec.max_positions == d["max_position_embeddings"]


def test_defaults_and_head_dim():
    d = copy.deepcopy(TINY["A"])
    for k in ("num_key_value_heads", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        d.pop(k)
    cfg = Qwen2Config.from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6 and not cfg.tie_word_embeddings
    assert cfg.head_dim == 16
    assert Qwen2Config.from_dict(TINY["C"]).head_dim == 48


def test_windows_by_layer():
    cfg = Qwen2Config.from_dict(TINY["C"])
    assert [cfg.layer_window(i) for i in range(4)] == [0, 0, 40, 40]
    d = dict(TINY["C"], layer_types=["sliding_attention", "full_attention"] * 2)
    cfg = Qwen2Config.from_dict(d)
    assert [cfg.layer_window(i) for i in range(4)] == [40, 0, 40, 0]
    d = dict(TINY["C"], use_sliding_window=False)
    assert [l.mixer.window for l in Qwen2Config.from_dict(d).to_spec().layers] == [0] * 4


def test_eos_forms():
    assert Qwen2Config.from_dict(TINY["A"]).eos_token_ids == (7,)
    assert Qwen2Config.from_dict(TINY["B"]).eos_token_ids == (998, 999)
    assert Qwen2Config.from_dict(TINY["C"]).eos_token_ids == ()


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "max_position_embeddings"])
def test_missing_key_is_named(key):
    d = copy.deepcopy(TINY["B"])
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("key,value", [
    ("hidden_size", "64"), ("hidden_size", 0), ("num_hidden_layers", 2.5), ("rms_norm_eps", -1.0),
    ("rope_theta", 0), ("tie_word_embeddings", 1), ("num_key_value_heads", 4), ("head_dim", 15),
    ("eos_token_id", "x"), ("vocab_size", True)])
def test_invalid_value_is_named(key, value):
    d = dict(copy.deepcopy(TINY["B"]), **{key: value})
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


def test_unsupported_options():
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen2Config.from_dict(dict(TINY["A"], rope_scaling={"type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen2Config.from_dict(dict(TINY["A"], hidden_act="gelu"))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(dict(TINY["A"], use_sliding_window=True))
    with pytest.raises(ConfigError, match="layer_types"):
        Qwen2Config.from_dict(dict(TINY["C"], layer_types=["full_attention"]))


def test_registry():
    assert lookup(TINY["A"]).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        lookup(dict(TINY["A"], architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        lookup({k: v for k, v in TINY["A"].items() if k != "architectures"})
    register_architecture("TestOnlyArch", Qwen2Config.from_dict, Qwen2Config.to_spec)
    try:
        assert lookup(dict(TINY["A"], architectures=["TestOnlyArch"])).name == "TestOnlyArch"
    finally:
        from sonicboom_b200.config import ARCHITECTURES
        ARCHITECTURES.pop("TestOnlyArch")


def test_round_trip_and_file(tmp_path):
    for d in TINY.values():
        cfg = Qwen2Config.from_dict(d)
        assert Qwen2Config.from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    assert read_config_json(tmp_path)["hidden_size"] == 192
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        read_config_json(tmp_path)
    with pytest.raises(ConfigError, match="config.json"):
        read_config_json(tmp_path / "nowhere")


def test_schedule_validation():
    import dataclasses
    _, spec = spec_from_config_dict(TINY["A"])
    ok = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, 1)))
    ok.validate()
    for bad in [(ScheduleEntry(0), ScheduleEntry(5)), (ScheduleEntry(0, 0),),
                (ScheduleEntry(0), ScheduleEntry(1, 0), ScheduleEntry(1, 1))]:
        with pytest.raises(ConfigError):
            dataclasses.replace(spec, schedule=bad).validate()
