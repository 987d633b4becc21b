"""Typed configuration and the architecture registry."""
import json

import pytest

from pih_b200.config import (Qwen3Config, config_from_dict, load_config, register_architecture,
                             registered_architectures)


def test_every_size_comes_from_config_json(tiny_configs):
    for name, raw in tiny_configs.items():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, Qwen3Config)
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
                    "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
            assert getattr(cfg, key) == raw[key], (name, key)
        spec = cfg.model_spec()
        assert len(spec.blocks) == raw["num_hidden_layers"] == len(spec.schedule)
        a = spec.blocks[0].mixer
        assert (a.heads, a.kv_heads, a.head_dim) == (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert a.q_size == cfg.q_projection_size and a.kv_size == cfg.kv_projection_size
        assert a.qk_norm_eps == raw["rms_norm_eps"] and a.position.theta == raw["rope_theta"]
        assert abs(a.scale - raw["head_dim"] ** -0.5) < 1e-12
        assert spec.blocks[0].ffn.intermediate == raw["intermediate_size"]
        assert spec.tie_embeddings == raw["tie_word_embeddings"]


def test_window_layers_follow_max_window_layers(tiny_configs):
    spec = config_from_dict(tiny_configs["B"]).model_spec()
    assert [b.mixer.window for b in spec.blocks] == [None, 24, 24]
    assert all(b.mixer.window is None for b in config_from_dict(tiny_configs["A"]).model_spec().blocks)


def test_head_dim_defaults_to_hidden_over_heads(tiny_configs):
    raw = dict(tiny_configs["A"])
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 16


def test_roundtrip_through_a_folder(tmp_path, tiny_configs):
    cfg = config_from_dict(tiny_configs["B"])
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(str(tmp_path)) == cfg


@pytest.mark.parametrize("change,match", [
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"architectures": []}, "exactly one"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"torch_dtype": "float16"}, "torch_dtype"),
    ({"eos_token_id": 100000}, "outside the vocabulary"),
    ({"eos_token_id": [2, 100000]}, "outside the vocabulary"),
    ({"eos_token_id": [2, "x"]}, "eos_token_id"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_bad_configurations_are_refused(tiny_configs, change, match):
    raw = dict(tiny_configs["A"])
    raw.update(change)
    with pytest.raises(ValueError, match=match):
        config_from_dict(raw)


def test_several_end_of_sequence_ids(tmp_path, tiny_configs):
    cfg = config_from_dict(dict(tiny_configs["A"], eos_token_id=[2, 5]))
    assert cfg.model_spec().eos_token_ids == (2, 5)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(str(tmp_path)) == cfg
    one = config_from_dict(dict(tiny_configs["A"], eos_token_id=7))
    assert one.model_spec().eos_token_ids == (7,)


def test_missing_key_is_an_error(tiny_configs):
    for key in ("hidden_size", "rope_theta", "rms_norm_eps", "vocab_size", "num_hidden_layers"):
        raw = dict(tiny_configs["A"])
        del raw[key]
        with pytest.raises(ValueError, match=key):
            config_from_dict(raw)


def test_registry_names_and_double_registration():
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ValueError, match="already registered"):
        @register_architecture("Qwen3ForCausalLM")
        class Other:
            pass
