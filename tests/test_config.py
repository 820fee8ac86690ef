"""Configuration and registry (no GPU): keys, refusals, bounds, windows, round trip."""
import json

import pytest

from mormot2_ai_b200 import ConfigError, Qwen3Config, config_of_folder, register_architecture
from mormot2_ai_b200.config import family_of
from tests.conftest import tiny_a, tiny_b


def base_doc():
    return tiny_a().to_dict()


def test_round_trip_and_derived_sizes():
    for make in (tiny_a, tiny_b):
        cfg = make()
        again = Qwen3Config.from_dict(cfg.to_dict())
        assert again == cfg
        assert cfg.q_width == cfg.num_attention_heads * cfg.head_dim
        assert cfg.kv_width == cfg.num_key_value_heads * cfg.head_dim
        assert cfg.group * cfg.num_key_value_heads == cfg.num_attention_heads
    assert tiny_b().q_width != tiny_b().hidden_size


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "max_position_embeddings",
                                 "rms_norm_eps", "hidden_act", "head_dim"])
def test_required_keys(key):
    doc = base_doc()
    del doc[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(doc)


@pytest.mark.parametrize("change,match", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "bias"),
    ({"mlp_bias": True}, "bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6}}, "rope_type"),
    ({"model_type": "llama"}, "model_type"),
    ({"num_key_value_heads": 3}, "shape"),
    ({"head_dim": 15}, "shape"),
    ({"head_dim": 2048}, "shape"),
    ({"rms_norm_eps": 0}, "shape"),
    ({"rms_norm_eps": 2.0}, "shape"),
    ({"rope_theta": 1.0}, "shape"),
    ({"vocab_size": 0}, "shape"),
    ({"num_hidden_layers": 0}, "shape"),
    ({"num_hidden_layers": 2000}, "shape"),
    ({"max_position_embeddings": 1 << 25}, "shape"),
    ({"use_sliding_window": True, "sliding_window": -4}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, "layer types"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "slides without"),
    ({"use_sliding_window": True, "sliding_window": 8,
      "layer_types": ["full_attention", "chunked_attention"]}, "layer type"),
    ({"vocab_size": "many"}, "integer"),
])
def test_refusals(change, match):
    doc = base_doc()
    doc.update(change)
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict(doc)


def test_rope_theta_places():
    doc = base_doc()
    theta = doc.pop("rope_theta")
    with pytest.raises(ConfigError):
        Qwen3Config.from_dict(doc)       # no theta anywhere: out of bounds
    doc["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "default"}
    assert Qwen3Config.from_dict(doc).rope_theta == 5e5
    doc2 = base_doc()
    doc2["rope_scaling"] = {}
    assert Qwen3Config.from_dict(doc2).rope_theta == theta


def test_windows_follow_the_reference_rules():
    doc = base_doc()
    doc["num_hidden_layers"] = 4
    # no window unless use_sliding_window, whatever else the file says
    doc.update({"use_sliding_window": False, "sliding_window": 8, "max_window_layers": 1})
    assert Qwen3Config.from_dict(doc).layer_windows == (0, 0, 0, 0)
    # then the layers from max_window_layers on
    doc["use_sliding_window"] = True
    assert Qwen3Config.from_dict(doc).layer_windows == (0, 8, 8, 8)
    # max_window_layers defaults to 28: no layer of a small model slides
    del doc["max_window_layers"]
    assert Qwen3Config.from_dict(doc).layer_windows == (0, 0, 0, 0)
    # sliding_window defaults to 4096
    del doc["sliding_window"]
    doc["max_window_layers"] = 2
    assert Qwen3Config.from_dict(doc).layer_windows == (0, 0, 4096, 4096)
    # null: no window
    doc["sliding_window"] = None
    assert Qwen3Config.from_dict(doc).layer_windows == (0, 0, 0, 0)
    # layer_types win over max_window_layers
    doc["sliding_window"] = 16
    doc["layer_types"] = ["sliding_attention", "full_attention", "full_attention",
                          "sliding_attention"]
    assert Qwen3Config.from_dict(doc).layer_windows == (16, 0, 0, 16)


def test_tied_default_is_false():
    doc = base_doc()
    del doc["tie_word_embeddings"]
    assert Qwen3Config.from_dict(doc).tie_word_embeddings is False


def test_registry_by_architecture_and_model_type(tmp_path):
    doc = base_doc()
    assert family_of(doc) is Qwen3Config
    del doc["architectures"]
    assert family_of(doc) is Qwen3Config            # by model_type
    doc["architectures"] = ["SomethingElse"]
    assert family_of(doc) is Qwen3Config            # unknown name, known model_type
    doc["model_type"] = "other"
    with pytest.raises(ConfigError, match="SomethingElse"):
        family_of(doc)
    del doc["architectures"]
    with pytest.raises(ConfigError, match="other"):
        family_of(doc)
    (tmp_path / "config.json").write_text(json.dumps(base_doc()))
    assert config_of_folder(str(tmp_path)) == tiny_a()
    with pytest.raises(ConfigError, match="cannot read"):
        config_of_folder(str(tmp_path / "missing"))


def test_first_registration_wins():
    class Other:
        pass
    register_architecture(Other, "Qwen3ForCausalLM", "qwen3")
    assert family_of(base_doc()) is Qwen3Config


def test_model_spec_is_data():
    spec = tiny_b().to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 2]
    assert [r.cache_line for r in spec.schedule] == [0, 1, 2]
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 24, 0]
    assert spec.layers[0].mixer.kind == "gqa_attention"
    assert spec.layers[0].feed_forward.kind == "swiglu"
    assert spec.head.params["tied"] is False and tiny_a().to_model_spec().head.params["tied"]
    assert spec.positions["rope"].params["theta"] == 1e6
